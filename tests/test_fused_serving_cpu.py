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
