"""Host-side scheduler of the fused disaggregated serving path: admission, mixed prompt / decode micro-batches, slots
and block-table rows from the native block manager, completion."""
from disagmoe_b200 import disagmoe_c as C
from disagmoe_b200.parallel.serving import FusedScheduler


def _fake_model(plans):
    # "next token" = (token id of the emitting row + position) % 97: depends on what the scheduler staged
    return [[(i + p) % 97 for i, p in zip(pl.ids, pl.pos)] for pl in plans]


def test_mixed_prefill_decode_micro_batches():
    bm = C.BlockManager(16, 64, 0, 8)
    s = FusedScheduler(bm, 16, n_mb=2, max_seqs_per_mb=2, max_tokens_per_mb=48, max_prefill_tokens_per_mb=40)
    s.add_request(0, list(range(10, 30)), 3, t_arrival=0.0)       # 20 prompt tokens
    s.add_request(1, list(range(50, 55)), 2, t_arrival=0.0)       # 5
    s.add_request(2, list(range(60, 78)), 2, t_arrival=5.0)       # arrives later
    assert s.has_work(0.0) and s.num_unfinished() == 3
    plans = s.build(0.0)
    # request 0 goes to micro-batch 0, request 1 to the emptier micro-batch 1; request 2 has not arrived
    assert [len(p) for p in plans] == [20, 5]
    p0 = plans[0]
    assert p0.ids == list(range(10, 30)) and p0.pos == list(range(20)) and len(set(p0.rows)) == 1
    blocks = bm.get_seq_block_list(0)
    assert p0.slots == [blocks[i // 16] * 16 + i % 16 for i in range(20)]
    assert [(r, q.req_id, g) for r, q, g in p0.emit] == [(19, 0, 20)]
    out = s.commit(plans, _fake_model(plans), now=1.0)
    assert sorted(r for r, _ in out) == [0, 1]
    assert s.running[0][0].length == 20 and s.running[1][1].length == 5
    # second iteration: both decode one token; request 2 still in the future
    plans = s.build(2.0)
    assert [len(p) for p in plans] == [1, 1]
    assert plans[0].pos == [20] and plans[0].ids == [s.running[0][0].last_token]
    assert plans[0].slots == [bm.slot_of(0, 20)]
    s.commit(plans, _fake_model(plans), now=2.5)
    assert 1 in s.finished and len(s.finished[1].outputs) == 2 and not bm.has_seq_block_list(1)
    # third iteration: request 2 arrives and joins the emptier micro-batch next to request 0's decode token
    plans = s.build(6.0)
    assert sorted(len(p) for p in plans) == [1, 18]
    s.commit(plans, _fake_model(plans), now=6.5)
    assert 0 in s.finished and len(s.finished[0].outputs) == 3
    plans = s.build(7.0)
    s.commit(plans, _fake_model(plans), now=7.5)
    assert s.num_unfinished() == 0 and not s.has_work(8.0)
    assert bm.num_free_blocks() == 64
    assert s.finished[2].t_tokens == [6.5, 7.5]


def test_admission_respects_limits():
    bm = C.BlockManager(16, 4, 0, 8)           # 4 blocks = 64 tokens of KV
    s = FusedScheduler(bm, 16, n_mb=2, max_seqs_per_mb=1, max_tokens_per_mb=40)
    for i in range(4):
        s.add_request(i, [1] * 20, 2, t_arrival=0.0)
    plans = s.build(0.0)
    # one sequence per micro-batch (max_seqs_per_mb), 2 blocks each: the KV pool is then full
    assert [len(p) for p in plans] == [20, 20] and len(s.waiting) == 2
    s.commit(plans, _fake_model(plans), 0.1)
    plans = s.build(0.2)
    assert [len(p) for p in plans] == [1, 1]
    s.commit(plans, _fake_model(plans), 0.3)     # both finish (2 tokens) and release their blocks
    plans = s.build(0.4)
    assert [len(p) for p in plans] == [20, 20] and not s.waiting


# ---- the host protocol of a whole job as CPU processes (gloo): control all-reduce, TP plan sharing, results ----------
class _FakeAttention:
    """Stands in for the GPU side of an attention rank: same buffers, next token = f(token, position)."""

    def __init__(self, srv, vocab):
        import torch
        z = lambda n, dt=torch.int32: torch.zeros(n, dtype=dt)
        self.mb = [dict(ids=z(srv.cap), positions=z(srv.cap), ctx_len=z(srv.cap), bt_row=z(srv.cap),
                        slots=z(srv.cap, torch.int64), next_ids=z(srv.cap)) for _ in range(srv.n_mb)]
        self.block_tables = torch.zeros(2 * srv.cap + 8, 64, dtype=torch.int32)
        self.layers = []
        self.active = [srv.cap] * srv.n_mb
        self.vocab = vocab
        self.seen_patches = 0

    def set_active(self, m, T):
        self.active[m] = T

    def iteration(self):
        for m, d in enumerate(self.mb):
            T = self.active[m]
            d["next_ids"][:T] = (d["ids"][:T] * 7 + d["positions"][:T] * 3 + 1) % self.vocab


class _FakeExpert:
    def iteration(self):
        pass


def _serving_worker(rank, world, n_attn, tp, port, q):
    import os
    import torch
    import torch.distributed as dist
    from disagmoe_b200.config import tiny_config
    from disagmoe_b200.parallel.serving import FusedServingRank
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = tiny_config
    mk = lambda role, srv: _FakeAttention(srv, cfg.vocab_size) if role == "attention" else _FakeExpert()
    srv = FusedServingRank(cfg, world, rank, 0, n_attn, tp, max_seqs_per_mb=4, max_tokens_per_mb=64, num_blocks=128,
                           host_only_runner=mk)
    groups = n_attn // tp
    g = torch.Generator().manual_seed(0)
    reqs = [(i, torch.randint(0, cfg.vocab_size, (int(torch.randint(3, 30, (1,), generator=g)),), generator=g).tolist(),
             int(torch.randint(2, 9, (1,), generator=g)), 0.002 * i) for i in range(20)]
    mine = [r for r in reqs if srv.is_leader and r[0] % groups == rank // tp]
    res = srv.serve(mine, time_limit=60)
    # a TP member must have been handed exactly the block-table entries of its leader
    res["table_sum"] = int(srv.runner.block_tables.sum()) if srv.is_attn else -1
    res["slo"] = [(s.req_id, len(s.t_tokens)) for s in res["slo"]]
    q.put((rank, res, reqs if rank == 0 else None))
    dist.destroy_process_group()


def _expected_tokens(prompt, n_out, vocab):
    out, tok, pos = [], prompt[-1], len(prompt) - 1
    for _ in range(n_out):
        tok = (tok * 7 + pos * 3 + 1) % vocab
        out.append(tok)
        pos += 1
    return out


def _run_job(world, n_attn, tp, port):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_serving_worker, args=(r, world, n_attn, tp, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    got = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(timeout=30)
        assert p.exitcode == 0
    return {r: res for r, res, _ in got}, next(x for _, _, x in got if x is not None)


def test_host_protocol_two_dp_groups_cpu():
    from disagmoe_b200.config import tiny_config
    res, reqs = _run_job(world=3, n_attn=2, tp=1, port=29741)
    outs = {**res[0]["outputs"], **res[1]["outputs"]}
    assert len(outs) == 20 and "outputs" not in res[2]
    for rid, prompt, n_out, _ in reqs:
        assert outs[rid] == _expected_tokens(prompt, n_out, tiny_config.vocab_size), rid
    assert res[0]["iterations"] == res[1]["iterations"] == res[2]["iterations"] > 0
    # every attention rank logs its iterations; the benchmark turns the logs into a Chrome trace
    assert len(res[0]["step_log"]) == res[0]["iterations"] and not res[2]["step_log"]
    import gzip
    import json
    import os
    import tempfile
    from benchmark.serve_fused import write_trace
    path = write_trace(list(res.values()), os.path.join(tempfile.mkdtemp(), "t.json.gz"))
    ev = json.load(gzip.open(path, "rt"))
    assert len(ev) == 2 * res[0]["iterations"] and {e["pid"] for e in ev} == {0, 1}
    assert all(e["dur"] >= 0 and len(e["args"]["rows_per_micro_batch"]) == 2 for e in ev)


def test_host_protocol_tensor_parallel_group_cpu():
    from disagmoe_b200.config import tiny_config
    res, reqs = _run_job(world=4, n_attn=2, tp=2, port=29742)
    outs = res[0]["outputs"]
    assert len(outs) == 20 and "outputs" not in res[1]
    for rid, prompt, n_out, _ in reqs:
        assert outs[rid] == _expected_tokens(prompt, n_out, tiny_config.vocab_size), rid
    assert res[0]["table_sum"] == res[1]["table_sum"] > 0
    assert len({res[r]["iterations"] for r in range(4)}) == 1


def test_tight_kv_pool_never_runs_dry():
    """Admission keeps the blocks free that the running sequences will still grow into: with a pool far smaller than
    the total demand, decode steps never hit 'out of KV blocks' and every request finishes."""
    import random
    bm = C.BlockManager(16, 24, 0, 64)
    s = FusedScheduler(bm, 16, n_mb=2, max_seqs_per_mb=8, max_tokens_per_mb=256)
    rnd = random.Random(0)
    for i in range(30):
        s.add_request(i, [1] * rnd.randint(5, 60), rnd.randint(10, 70), 0.0)
    steps = 0
    while s.num_unfinished():
        plans = s.build(1.0)
        assert any(len(p) for p in plans), "nothing runnable although requests are pending"
        s.commit(plans, [[7] * len(p) for p in plans], 1.0)
        steps += 1
        assert steps < 5000
    assert len(s.finished) == 30 and bm.num_free_blocks() == 24


def test_long_prompt_is_prefilled_in_chunks_next_to_decode_rows():
    """A prompt longer than the per-iteration prompt budget is split over iterations: positions continue where the last
    chunk stopped, only the last chunk samples, and the sequences that are decoding get their token every iteration."""
    bm = C.BlockManager(16, 64, 0, 8)
    s = FusedScheduler(bm, 16, n_mb=1, max_seqs_per_mb=4, max_tokens_per_mb=40, max_prefill_tokens_per_mb=32)
    s.add_request(0, list(range(100, 105)), 6, t_arrival=0.0)      # short: decoding from the 2nd iteration on
    s.add_request(1, list(range(200, 290)), 2, t_arrival=0.0)      # 90 prompt tokens: 27 + 32 + 31
    plans = s.build(0.0)
    p = plans[0]
    assert len(p) == 32 and p.ids[:5] == list(range(100, 105)) and p.ids[5:] == list(range(200, 227))
    assert [(r, q.req_id, g) for r, q, g in p.emit] == [(4, 0, 5), (-1, 1, 27)]
    out = s.commit(plans, _fake_model(plans), 0.1)
    assert [r for r, _ in out] == [0] and s.running[0][1].length == 27 and not s.running[0][1].outputs
    plans = s.build(0.2)                                               # 1 decode row + the next 32 prompt rows
    p = plans[0]
    assert len(p) == 33 and p.pos[0] == 5 and p.pos[1:] == list(range(27, 59)) and p.ids[1] == 227
    blocks = bm.get_seq_block_list(1)
    assert p.slots[1:] == [blocks[i // 16] * 16 + i % 16 for i in range(27, 59)]
    assert [(r, q.req_id, g) for r, q, g in p.emit] == [(0, 0, 1), (-1, 1, 32)]
    s.commit(plans, _fake_model(plans), 0.3)
    plans = s.build(0.4)                                               # last chunk: 31 rows, its last row samples
    p = plans[0]
    assert len(p) == 32 and p.pos[1:] == list(range(59, 90))
    assert [(r, q.req_id, g) for r, q, g in p.emit] == [(0, 0, 1), (31, 1, 31)]
    out = s.commit(plans, _fake_model(plans), 0.5)
    assert sorted(r for r, _ in out) == [0, 1] and s.running[0][1].length == 90
    while s.num_unfinished():
        plans = s.build(1.0)
        s.commit(plans, _fake_model(plans), 1.0)
    assert len(s.finished[0].outputs) == 6 and len(s.finished[1].outputs) == 2 and bm.num_free_blocks() == 64


def test_scheduler_invariants_on_random_streams():
    """Random request streams against random budgets: every iteration respects the row and prompt budgets and the
    per-micro-batch sequence limit, every sequence's positions advance without gaps, only the last prompt row and the
    decode rows sample, every request finishes with its length, and no KV block leaks."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=40, deadline=None)
    @given(st.integers(0, 10_000), st.integers(1, 3), st.integers(1, 6), st.integers(24, 96), st.integers(16, 64))
    def run(seed, n_mb, max_seqs, max_tokens, max_prefill):
        import random
        rnd = random.Random(seed)
        bm = C.BlockManager(16, 96, 0, 64)
        s = FusedScheduler(bm, 16, n_mb, max_seqs, max(max_tokens, max_seqs + 16), max_prefill)
        reqs = {i: (rnd.randint(1, 120), rnd.randint(1, 12), rnd.random() * 3) for i in range(rnd.randint(1, 14))}
        for i, (n_in, n_out, at) in sorted(reqs.items(), key=lambda kv: kv[1][2]):
            s.add_request(i, [rnd.randrange(1000) for _ in range(n_in)], n_out, at)
        next_pos = {i: 0 for i in reqs}
        now, steps = 0.0, 0
        while s.num_unfinished():
            now += 0.25
            plans = s.build(now)
            for m, p in enumerate(plans):
                assert len(p) <= s.max_tokens and len(s.running[m]) <= max_seqs
                assert len(p.ids) == len(p.pos) == len(p.rows) == len(p.slots)
                sampled = {row for row, _, _ in p.emit if row >= 0}
                assert len(sampled) == len([e for e in p.emit if e[0] >= 0])
                prompt_rows = 0
                cursor = 0
                for row, q, grown in p.emit:                       # emit entries are in row order
                    first = (row - grown + 1) if row >= 0 else cursor
                    for k in range(grown):
                        assert p.pos[first + k] == next_pos[q.req_id] + k
                    if not (row >= 0 and grown == 1 and q.length >= len(q.prompt)):
                        prompt_rows += grown
                    next_pos[q.req_id] += grown
                    cursor = first + grown
                assert prompt_rows <= max_prefill
            s.commit(plans, [[1] * len(p) for p in plans], now)
            steps += 1
            assert steps < 4000
        assert set(s.finished) == set(reqs)
        for i, (n_in, n_out, _) in reqs.items():
            assert len(s.finished[i].outputs) == n_out and s.finished[i].length == n_in + n_out - 1
        assert bm.num_free_blocks() == 96

    run()


def test_eos_ends_a_request_when_not_ignored():
    from disagmoe_b200.utils.constants import EOS_TOKEN_ID
    bm = C.BlockManager(16, 16, 0, 4)
    s = FusedScheduler(bm, 16, 1, 2, 64, ignore_eos=False)
    s.add_request(0, [5, 6, 7], 10, 0.0)
    plans = s.build(0.0)
    s.commit(plans, [[9] * len(plans[0])], 0.1)                 # first token: not EOS
    plans = s.build(0.2)
    s.commit(plans, [[EOS_TOKEN_ID]], 0.3)                      # second token: EOS
    assert s.finished[0].outputs == [9, EOS_TOKEN_ID] and s.num_unfinished() == 0 and bm.num_free_blocks() == 16


def test_request_assignment_balances_groups_deterministically():
    import random
    from benchmark.serve_fused import assign_requests
    rnd = random.Random(0)
    reqs = [(i, [0] * rnd.randint(100, 1000), rnd.randint(50, 500), i * 0.05) for i in range(200)]
    owner = assign_requests(reqs, 4)
    assert owner == assign_requests(list(reversed(reqs)), 4)          # a function of the workload, not of its order
    work = [0] * 4
    for rid, prompt, n_out, _ in reqs:
        work[owner[rid]] += len(prompt) + n_out
    assert max(work) / min(work) < 1.5                                  # total work stays roughly even too
    assert set(assign_requests(reqs, 1).values()) == {0}


def test_serve_fused_script_host_only_dry_run(tmp_path):
    """benchmark/serve_fused.py end to end as CPU processes (2 attention groups + 1 expert rank): workload, request
    assignment, lock-step serving with chunked prefill, result collection, metrics file, Chrome trace."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out, trace = tmp_path / "m.jsonl", tmp_path / "t.json.gz"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "3", "--master-addr",
           "127.0.0.1", "--master-port", "29771", os.path.join(root, "benchmark", "serve_fused.py"), "--host-only",
           "--model", "tiny", "--n-attn", "2", "-r", "300", "-n", "30", "--min-input-len", "5", "-i", "60",
           "--min-output-len", "2", "-o", "9", "--max-seqs-per-mb", "4", "--max-tokens-per-mb", "48",
           "--max-prefill-tokens-per-mb", "20", "--num-blocks", "256", "--time-limit", "60", "--check", "-f", str(out),
           "--trace", str(trace)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    lines = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert next(l for l in lines if "check_requests_exact" in l) == {"check_requests_exact": 30, "requests": 30}
    info = next(l for l in lines if "iterations" in l)
    assert info["requests_finished"] == 30 and info["kernel_status"] == 0
    row = json.loads(out.read_text().strip().splitlines()[-1])
    assert row["token_throughput"] > 0 and trace.exists()


def test_native_scheduler_builds_the_same_plans_as_the_python_statement():
    """The C++ serving scheduler (csrc/runtime/fused_scheduler.cpp) against the Python statement of the same policy on
    random request streams: identical plans (ids, positions, block-table rows, slots, emit lists) every iteration,
    identical tokens committed, identical finish order."""
    import random
    from disagmoe_b200.parallel.serving import PyFusedScheduler
    for seed in range(25):
        rnd = random.Random(seed)
        n_mb, max_seqs = rnd.randint(1, 3), rnd.randint(1, 6)
        max_tokens, max_prefill = max(rnd.randint(24, 96), max_seqs + 16), rnd.randint(16, 64)
        bms = [C.BlockManager(16, 96, 0, 64) for _ in range(2)]
        a = C.FusedScheduler(bms[0], 16, n_mb, max_seqs, max_tokens, max_prefill, False)
        b = PyFusedScheduler(bms[1], 16, n_mb, max_seqs, max_tokens, max_prefill, False)
        reqs = [(i, [rnd.randrange(1000) for _ in range(rnd.randint(1, 120))], rnd.randint(1, 12), rnd.random() * 3)
                for i in range(rnd.randint(1, 14))]
        for r in sorted(reqs, key=lambda r: r[3]):
            a.add_request(*r)
            b.add_request(*r)
        now = 0.0
        while b.num_unfinished():
            now += 0.25
            assert a.has_work(now) == b.has_work(now) and a.num_unfinished() == b.num_unfinished()
            pa, pb = a.build(now), b.build(now)
            for x, y in zip(pa, pb):
                assert list(x.ids) == y.ids and list(x.pos) == list(y.pos) and list(x.rows) == y.rows
                assert list(x.slots) == list(y.slots)
                assert [(r, q.req_id, g) for r, q, g in x.emit] == [(r, q.req_id, g) for r, q, g in y.emit]
            toks = [[rnd.choice([2, 5, 9]) for _ in range(len(p))] for p in pb]      # 2 = EOS: early finishes too
            assert a.commit(pa, toks, now) == b.commit(pb, toks, now)
            assert [sorted(r) for r in a.running] == [sorted(r) for r in b.running]
        assert a.num_unfinished() == 0 and set(a.finished) == set(b.finished)
        for i in b.finished:
            assert list(a.finished[i].outputs) == b.finished[i].outputs and a.finished[i].length == b.finished[i].length
        assert bms[0].num_free_blocks() == bms[1].num_free_blocks() == 96


def test_layer_striping_shape_assigns_contiguous_layer_blocks():
    """DisaggShape(stripes=A): contiguous blocks of ceil(L / A) layers per pipeline stage, the LM head (layer L) on the
    last stage, and an arena layout that adds one residual hand-off buffer and flag per micro-batch."""
    import pytest
    from disagmoe_b200.parallel.disagg import DisaggShape, build_layout
    s = DisaggShape(3, 2, 2, 8, 2, 256, 8, stripes=3, num_layers=8)
    assert [s.layer_owner(l) for l in range(9)] == [0, 0, 0, 1, 1, 1, 2, 2, 2]
    assert DisaggShape(2, 2, 2, 8, 2, 256, 8).layer_owner(3) == -1
    lay, plain = build_layout(s), build_layout(DisaggShape(3, 2, 2, 8, 2, 256, 8))
    assert {"ho_resid0", "ho_flag0", "ho_resid1", "ho_flag1"} <= set(lay.entries) and "ho_resid0" not in plain.entries
    assert lay.entries["ho_resid0"][1] == 8 * 256 * 2
    with pytest.raises(AssertionError):
        DisaggShape(4, 2, 2, 8, 2, 256, 8, tp=2, stripes=4, num_layers=8)      # no TP inside a stage
    with pytest.raises(AssertionError):
        DisaggShape(4, 2, 2, 8, 2, 256, 8, stripes=2, num_layers=8)            # one pipeline over all attention GPUs


def test_prefill_tile_builder_finds_prompt_runs_and_leaves_the_rest():
    """build_prefill_tiles (host side of the tiled causal attention): runs of consecutive positions of one sequence
    with at least min_len rows become tiles of at most tile_tokens rows; decode rows and short runs stay uncovered."""
    import torch
    from disagmoe_b200.ops.functional import build_prefill_tiles
    #        decode rows   | prompt of seq 7: positions 10..29        | short run of seq 9 | prompt chunk of seq 3
    rows = [0, 1, 2] + [7] * 20 + [9] * 3 + [3] * 9
    pos = [55, 12, 80] + list(range(10, 30)) + [0, 1, 2] + list(range(100, 109))
    tiles, covered = build_prefill_tiles(rows, pos, tile_tokens=16, min_len=8)
    assert tiles.dtype == torch.int32 and tiles.tolist() == [[3, 16, 7, 10], [19, 4, 7, 26], [26, 9, 3, 100]]
    assert covered.tolist() == [False] * 3 + [True] * 20 + [False] * 3 + [True] * 9
    # a break in the positions splits a run even inside one sequence; nothing to do for an empty batch
    tiles2, cov2 = build_prefill_tiles([4] * 16, list(range(8)) + list(range(20, 28)), tile_tokens=16)
    assert tiles2.tolist() == [[0, 8, 4, 0], [8, 8, 4, 20]] and bool(cov2.all())
    t0, c0 = build_prefill_tiles([], [], 16)
    assert t0.shape == (0, 4) and c0.numel() == 0
