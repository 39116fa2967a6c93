"""Property tests of the native wire types and the block manager against plain-Python restatements (random inputs)."""
from hypothesis import given, settings, strategies as st

from disagmoe_b200 import disagmoe_c as C
from disagmoe_b200.ops.memory import get_mappings_from_exp_ids


def _meta(req, exp, dp, prefill, pos, weights, hidden=8):
    m = C.Metadata([len(req), hidden])
    m.req_ids, m.exp_ids, m.attn_dp_ranks, m.init_prefill_lens, m.positions = req, exp, dp, prefill, pos
    m.topk_weights = weights
    return m


tokens = st.lists(st.tuples(st.integers(0, 500), st.integers(0, 7), st.integers(0, 3),
                            st.sampled_from([-1, 3, 9]), st.integers(0, 40), st.floats(0, 1, width=32)),
                  min_size=1, max_size=40)


@settings(max_examples=60, deadline=None)
@given(tokens)
def test_metadata_serialization_sort_and_slicing(toks):
    req, exp, dp, pre, pos, w = (list(x) for x in zip(*toks))
    m = _meta(req, exp, dp, pre, pos, w)
    r = C.Metadata.deserialize(m.serialize())
    assert (r.req_ids, r.exp_ids, r.attn_dp_ranks, r.init_prefill_lens, r.positions) == (req, exp, dp, pre, pos)
    assert all(abs(a - b) < 1e-6 for a, b in zip(r.topk_weights, w))
    # stable counting sort by expert: same permutation as the Python restatement, sizes and offsets agree
    merged, mapping = C.Metadata.merge_by_exp_ids([m])
    want_map, want_counts = get_mappings_from_exp_ids(exp, 8)
    assert mapping == want_map and merged.exp_ids == sorted(exp)
    assert [merged.req_ids[mapping[i]] for i in range(len(req))] == req
    assert m.get_expert_batch_sizes(8) == want_counts
    offs = merged.get_expert_offsets(8, list(range(8)))
    assert offs == [sum(want_counts[:e]) for e in range(9)]
    # slices and splits partition the tokens in order
    k = len(req) // 2
    a, b = m.split(k) if 0 < k < len(req) else (m.slice(0, 0), m)
    assert a.req_ids + b.req_ids == req
    # prefill order: by dp rank, prompt tokens before decode tokens, then request id; the returned order is a permutation
    order = m.sort_by_prefill_order()
    key = lambda i: (dp[i], 0 if pre[i] >= 0 else 1, req[i])
    assert sorted(order) == list(range(len(req)))
    got = list(zip(m.attn_dp_ranks, [0 if p >= 0 else 1 for p in m.init_prefill_lens], m.req_ids))
    assert got == sorted(got)
    assert sorted(got) == sorted(key(i) for i in range(len(req)))


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 4), st.lists(st.integers(0, 200), min_size=1, max_size=12))
def test_duplicate_and_shrink_topk_are_inverse(k, req):
    m = _meta(req, [-1] * len(req), [0] * len(req), [-1] * len(req), [0] * len(req), [1.0] * len(req))
    m.duplicate_topk(k)
    assert m.req_ids == [r for r in req for _ in range(k)]          # token-major: slot j of token i is row i*k + j
    assert m.topk_slots == list(range(k)) * len(req) and m.shape[0] == k * len(req)
    m.shrink_topk(k)
    assert m.req_ids == req and m.shape[0] == len(req)


ops = st.lists(st.tuples(st.sampled_from(["alloc", "grow", "release"]), st.integers(0, 9), st.integers(1, 70)),
               min_size=1, max_size=60)


@settings(max_examples=60, deadline=None)
@given(ops)
def test_block_manager_against_a_python_model(seq):
    """Random allocate / grow / release: blocks are never shared, counts match ceil(len / 16), slots follow the block
    list, every table change is reported exactly once, and releasing everything returns the pool."""
    bs, total = 16, 40
    bm = C.BlockManager(bs, total, 0, 16)
    lens = {}
    table = {}
    for op, sid, n in seq:
        if op == "alloc" and sid not in lens:
            if bm.can_allocate(n):
                bm.allocate(sid, n)
                lens[sid] = n
        elif op == "grow" and sid in lens:
            need = (lens[sid] + n + bs - 1) // bs - len(bm.get_seq_block_list(sid))
            if need <= bm.num_free_blocks():
                bm.append_tokens(sid, lens[sid], n)
                lens[sid] += n
        elif op == "release" and sid in lens:
            bm.release(sid)
            row = [r for r, s in table.items() if s[0] == sid]
            for r in row:
                del table[r]
            del lens[sid]
        for row, col, blk in bm.drain_updates():
            owner = next(s for s in lens if bm.row_of(s) == row)
            table.setdefault(row, (owner, {}))[1][col] = blk
        held = [b for s in lens for b in bm.get_seq_block_list(s)]
        assert len(held) == len(set(held)) and len(held) + bm.num_free_blocks() == total
        for s, n_tok in lens.items():
            blocks = bm.get_seq_block_list(s)
            assert len(blocks) == (n_tok + bs - 1) // bs
            assert bm.slot_of(s, n_tok - 1) == blocks[(n_tok - 1) // bs] * bs + (n_tok - 1) % bs
            # the reported patches reproduce the block list
            cols = table[bm.row_of(s)][1]
            assert [cols[c] for c in range(len(blocks))] == blocks
    bm.batch_release(list(lens))
    assert bm.num_free_blocks() == total and bm.num_seqs() == 0


def test_attention_pool_is_insensitive_to_arrival_order():
    """Partial rows of decode tokens arrive in random order and random groupings: a token is released exactly when its
    top-k + residual parts are all there, with every part in its own slot, whatever the order."""
    import random

    import torch
    K = 3                                                     # parts per token (top-2 + residual)
    C.set_inproc_transport(True)
    try:
        for seed in range(8):
            rnd = random.Random(seed)
            args = C.EngineArgs()
            args.local_id, args.has_attn, args.top_k = 710 + seed, True, K - 1
            args.attn_layer_ids = [1]
            args.parts_needed = {1: K}
            h = C.init_engine(args)
            p = h.attn_pool
            n_tok = rnd.randint(1, 9)
            parts = [(t, s) for t in range(n_tok) for s in range(K)]
            rnd.shuffle(parts)
            value = lambda t, s: torch.full((4,), float(10 * t + s))
            released, arrived = set(), {t: 0 for t in range(n_tok)}
            while parts:
                group = [parts.pop() for _ in range(min(len(parts), rnd.randint(1, 4)))]
                m = C.Metadata([len(group), 4])
                m.layer_id = 1
                m.req_ids = [100 + t for t, _ in group]
                m.exp_ids, m.attn_dp_ranks = [0] * len(group), [0] * len(group)
                m.init_prefill_lens, m.positions = [-1] * len(group), [7] * len(group)
                m.topk_slots = [s for _, s in group]
                p.process_batch(torch.stack([value(t, s) for t, s in group]), m, 0)
                for t, _ in group:
                    arrived[t] += 1
                b = p.fetch_attention_batch()
                complete = {t for t in arrived if arrived[t] == K} - released
                if not complete:
                    assert b.metadata is None
                    continue
                assert sorted(b.metadata.seq_ids) == sorted(100 + t for t in complete) and b.num_parts == K
                for row, sid in enumerate(b.metadata.seq_ids):
                    got = sorted(b.data[row, :, 0].tolist())
                    assert got == [float(10 * (sid - 100) + s) for s in range(K)]
                released |= complete
            assert released == set(range(n_tok)) and p.num_pending_tokens() == 0
            C.stop_engine(h)
    finally:
        C.set_inproc_transport(False)
