"""Native host runtime on CPU: serializer, metadata ops, block manager, layer schedulers, pools, channels, recorder,
placement and the DP scheduler."""
import asyncio

import pytest
import torch

from disagmoe_b200 import disagmoe_c as C
from disagmoe_b200.config import mixtral_config, tiny_config
from disagmoe_b200.ops.memory import get_mappings_from_exp_ids
from disagmoe_b200.scheduler.dpscheduler import get_dp_scheduler
from disagmoe_b200.utils.placement import ClusterConfig, get_model_placement


def _meta(req, exp, dp=None, prefill=None, pos=None, layer=0, hidden=8):
    m = C.Metadata([len(req), hidden])
    m.layer_id = layer
    m.req_ids, m.exp_ids = req, exp
    m.attn_dp_ranks = dp or [0] * len(req)
    m.init_prefill_lens = prefill or [-1] * len(req)
    m.positions = pos or [0] * len(req)
    return m


def test_in_module_self_tests():
    assert C.test_socket_p2p(7, 32)
    assert C.test_parallel_attn_scheduler(3, 12)
    assert C.test_recorder_threads(10) == 10


def test_metadata_roundtrip_and_ops():
    m = _meta([5, 6, 7, 8], [2, 0, 1, 0], dp=[1, 0, 1, 0], prefill=[-1, 4, -1, 4], pos=[9, 1, 3, 0])
    m.topk_weights = [0.1, 0.2, 0.3, 0.4]
    r = C.Metadata.deserialize(m.serialize())
    assert (r.req_ids, r.exp_ids, r.topk_weights[3], r.layer_id) == (m.req_ids, m.exp_ids, pytest.approx(0.4), 0)
    merged, mapping = C.Metadata.merge_by_exp_ids([m])
    assert merged.exp_ids == [0, 0, 1, 2] and merged.req_ids == [6, 8, 7, 5]
    assert mapping == get_mappings_from_exp_ids(m.exp_ids, 3)[0]
    assert m.get_expert_batch_sizes(3) == [2, 1, 1] and merged.get_expert_offsets(3, [1, 2]) == [0, 1, 2]
    order = m.sort_by_prefill_order()          # (dp rank, prefill first, req id)
    assert m.req_ids == [6, 8, 5, 7] and order == [2, 0, 3, 1]
    d = _meta([1, 2], [-1, -1])
    d.duplicate_topk(3)
    assert d.req_ids == [1, 1, 1, 2, 2, 2] and d.topk_slots == [0, 1, 2, 0, 1, 2] and d.shape[0] == 6
    d.shrink_topk(3)
    assert d.req_ids == [1, 2] and d.shape[0] == 2
    a, b = m.split(1)
    assert a.num_tokens() == 1 and b.num_tokens() == 3
    s = m.slice(1, 3)
    assert s.req_ids == [8, 5]
    m.step_layer()
    assert m.layer_id == 1


def test_tensor_batch_merge_sorts_rows_by_expert():
    t1, t2 = torch.arange(6.).view(3, 2), torch.arange(6., 10.).view(2, 2)
    b1 = C.TensorBatch(t1, _meta([1, 2, 3], [1, 0, 1], hidden=2))
    b2 = C.TensorBatch(t2, _meta([4, 5], [0, 2], hidden=2))
    out = C.TensorBatch.merge([b1, b2])
    assert out.metadata.exp_ids == [0, 0, 1, 1, 2] and out.metadata.req_ids == [2, 4, 1, 3, 5]
    assert out.data.tolist() == [[2, 3], [6, 7], [0, 1], [4, 5], [8, 9]]


def test_block_manager():
    bm = C.BlockManager(16, 10, 2)
    assert bm.num_free_blocks() == 12 and bm.can_allocate(160) and not bm.can_allocate(161)
    bm.allocate(1, 33)
    assert bm.get_seq_block_list(1) == [0, 1, 2] and bm.slot_of(1, 17) == 1 * 16 + 1
    bm.append_tokens(1, 48, 1)
    assert len(bm.get_seq_block_list(1)) == 4
    ups = bm.drain_updates()
    assert ups == [(0, 0, 0), (0, 1, 1), (0, 2, 2), (0, 3, 3)] and bm.drain_updates() == []
    rs = bm.step_decode([1], [64])
    assert rs == [0, 4 * 16] and len(bm.get_seq_block_list(1)) == 5
    am = C.AttentionBatchMetadata()
    am.seq_ids, am.init_prefill_lens, am.positions, am.attn_dp_ranks = [1, 2], [-1, 5], [65, 0], [0, 0]
    am.recount()
    assert (am.num_prefill_tokens, am.num_decode_tokens, am.num_prefill_seqs) == (1, 1, 1)
    bm.update_block_table(am, [65, 0])
    table, width = bm.prepare_block_table(am, [66, 1])
    assert width == 5 and table.numel() == 2 * 5 + 2 and int(table[-1]) == bm.get_seq_block_list(2)[0] * 16
    infos = C.prepare_batch_infos(am, [66, 1]).tolist()
    assert infos == [66, 1, 65, 0, 0, 66, 67]
    bm.batch_release([1, 2])
    assert bm.num_free_blocks() == 12 and bm.num_seqs() == 0
    with pytest.raises(RuntimeError):
        bm.allocate(3, 16 * 12)     # would eat the reserved blocks


def test_layer_scheduler_policies():
    def filled(policy, n=16):
        s = C.LayerScheduler(n, policy)
        for l, t in ((1, 3), (2, 10), (9, 12), (10, 1)):
            s.add_tokens_to_layer(l, t)
        return s
    assert filled("mbfs").schedule() == 9
    assert filled("flfs").schedule() == 1 and filled("bin").schedule() == 1
    s = filled("mbflfs")                       # blocks of 8: [0..7] holds 13 tokens, [8..15] holds 13 -> first wins
    assert s.schedule() == 1
    s = filled("mbflfs"); s.set_block_size(1)
    assert s.schedule() == 9
    s = filled("mbtfs"); s.add_tokens_to_layer(1, 1)
    assert s.schedule() == 1                   # two batches beat one larger batch
    assert C.LayerScheduler(4, "mbfs").schedule() == -1
    g = C.GroupLayerScheduler(4, 2)
    g.add_tokens_to_group(0, 1, 5); g.add_tokens_to_group(1, 1, 50); g.add_tokens_to_group(3, 0, 20)
    # look-ahead score = tokens of the cell + 0.8 * next layer + ...: (1,1) scores 50, (0,1) scores 5 + 0.8 * 50 = 45
    assert g.schedule() == g.cell(1, 1)
    assert g.schedule() == g.cell(3, 0) and g.schedule() == g.cell(0, 1) and g.schedule() == -1


def test_advanced_layer_scheduler_states():
    now = [0.0]
    s = C.AdvancedLayerScheduler(4, 2)
    s.set_clock(lambda: now[0])
    s.add_tokens_to_layer(0, 10)               # below the 256-token threshold: held
    s.add_tokens_to_layer(2, 300)              # ready at once
    assert s.schedule() == 2
    assert s.schedule() == 0                   # only a held layer left: it is served
    s.add_tokens_to_layer(1, 300); s.add_tokens_to_layer(3, 400)
    now[0] = 10.0
    assert s.schedule() == 3                   # both ready, larger look-ahead score first
    s.add_tokens_to_layer(3, 500)
    now[0] = 45.0                              # layer 1 has waited > 30 ms: urgent beats the bigger layer 3
    assert s.schedule() == 1


def test_attention_pool_waits_for_all_partials_and_orders_prompts():
    pool = C.init_engine  # noqa: F841  (module loads)
    args = C.EngineArgs()
    args.local_id, args.has_attn, args.top_k = 700, True, 2
    args.attn_layer_ids = [1]
    args.parts_needed = {1: 3}
    C.set_inproc_transport(True)
    h = C.init_engine(args)
    p = h.attn_pool
    rows = torch.arange(8.).view(2, 4)
    def partial(slot, reqs=(1, 1), pos=(0, 1)):
        m = _meta(list(reqs), [0, 0], prefill=[2, 2], pos=list(pos), layer=1, hidden=4)
        m.topk_slots = [slot] * 2
        p.process_batch(rows + slot, m, 0)
    partial(0); partial(2)
    assert p.fetch_attention_batch().metadata is None and p.num_pending_tokens() == 2
    partial(1)
    b = p.fetch_attention_batch()
    assert b.metadata.seq_ids == [1, 1] and b.metadata.positions == [0, 1] and b.num_parts == 3
    assert b.data.shape == (2, 3, 4) and torch.equal(b.data[:, 1], rows + 1)
    # prompt position 1 must not run before position 0
    for slot in range(3):
        m = _meta([2], [0], prefill=[2], pos=[1], layer=1, hidden=4); m.topk_slots = [slot]
        p.process_batch(rows[:1], m, 0)
    assert p.fetch_attention_batch().metadata is None
    for slot in range(3):
        m = _meta([2], [0], prefill=[2], pos=[0], layer=1, hidden=4); m.topk_slots = [slot]
        p.process_batch(rows[:1], m, 0)
    b = p.fetch_attention_batch()
    assert b.metadata.positions == [0, 1]
    C.stop_engine(h)
    C.set_inproc_transport(False)


def test_sampler_finish_rule_and_bookkeeping():
    C.set_inproc_transport(True)
    s = C.init_sampler(82, 2, 3, 1, [900], {0: 900}, False)
    s.set_request_output_len(7, 3)
    def feed(tok, pos):
        m = C.Metadata([1, 0]); m.req_ids, m.token_ids, m.positions, m.attn_dp_ranks = [7], [tok], [pos], [0]
        s.process_batch(m)
    feed(11, 4); feed(12, 5)
    assert s.num_finished() == 0 and s.get_output_tokens(7) == [11, 12]
    feed(2, 6)                                   # EOS (and the third token)
    st = s.fetch_finished_slo_stats()
    assert len(st) == 1 and st[0].req_id == 7 and len(st[0].t_tokens) == 3 and st[0].t_decode >= st[0].t_prefill
    assert s.fetch_finished_slo_stats() == [] and len(s.fetch_step_infos()) == 3
    s.set_request_output_len(8, 50)
    m = C.Metadata([1, 0]); m.req_ids, m.token_ids, m.positions, m.attn_dp_ranks = [8], [2], [3], [0]
    s.process_batch(m)                           # EOS ends request 8 although 49 tokens were left
    assert s.num_finished() == 2
    C.set_inproc_transport(False)


def test_placements():
    cfg = mixtral_config.clone(ep_size=4, dp_size=2, tp_size=1)
    p = get_model_placement(cfg, ClusterConfig(1, 8), "pipeline", 2, 1, True)
    assert sorted(p.attn) == [0, 1, 2, 3] and sorted(p.expert) == [4, 5, 6, 7]
    assert p.attn[0] == list(range(0, 32, 2)) and p.attn[2] == list(range(1, 32, 2))
    assert p.attn_dp_ranks == {0: 0, 1: 1, 2: 0, 3: 1}
    assert p.expert_rank_at(5) == 1 and {e for _, e in p.expert[5]} == {2, 3}
    assert set(p.out_device_ids[0]) == {4, 5, 6, 7} and set(p.in_device_ids[2]) == {4, 5, 6, 7}
    assert p.tokenizer in p.in_device_ids[0] and p.sampler in p.out_device_ids[4]
    tp = get_model_placement(mixtral_config.clone(ep_size=4, tp_size=4), ClusterConfig(1, 8), "pipeline", 1, 1)
    assert tp.device_groups[2] == [0, 1, 2, 3] and tp.is_worker_device(3) and not tp.is_worker_device(0)
    assert tp.sampler in tp.in_device_ids[0] and tp.sampler not in tp.in_device_ids.get(1, [])
    co = get_model_placement(mixtral_config.clone(ep_size=2), ClusterConfig(1, 2), "colocate")
    assert co.is_hybrid and co.attn[1] == list(range(32)) and co.expert_rank_at(1) == 1
    il = get_model_placement(tiny_config.clone(ep_size=2, tp_size=1), ClusterConfig(1, 6), "interleave")
    assert il.attn[0] == [0] and il.attn[3] == [1] and {l for l, _ in il.expert[4]} == {1}
    sg = get_model_placement(tiny_config.clone(ep_size=8), ClusterConfig(1, 18), "single")
    assert len(sg.attn) == 2 and len(sg.expert) == 16


def test_dp_scheduler_max_blocks_until_release():
    async def run():
        sch = get_dp_scheduler(2, 64, 16, "max")        # 4 blocks per sequence
        sch.start({0: 8, 1: 4})
        got = []
        for r in range(4):
            sch.put_request(lambda rid, rank: got.append((rid, rank)), r)
        await asyncio.sleep(0.05)
        assert got == [(0, 0), (1, 0), (2, 1)]          # request 3 waits: no replica has 4 free blocks
        sch.del_seq(1)
        await asyncio.sleep(0.05)
        assert got[-1] == (3, 0)
        await sch.terminate()
        rr = get_dp_scheduler(3, 64, 16, "RR")
        assert rr.schedule([10, 11, 12, 13]) == [0, 1, 2, 0]
    asyncio.run(run())


def test_native_module_keeps_the_reference_api_surface():
    """Every class / function name the reference binds in its disagmoe_c module (csrc/bindings.cpp:24-221) exists."""
    classes = ("MuHelper Scheduler AttentionScheduler MuDispatcher Tokenizer Sampler TopKSampler TensorBatch ChannelInfo "
               "Channel NcclGroupChannel TokenMetadata ParallelConfig AttentionBatch SloStat SamplerStepInfo "
               "AttentionBatchMetadata Metadata NcclChannel BlockManager TraceContext").split()
    functions = ("prepare_batch_infos permute_tokens_cuda recorder_output recorder_create range_push range_pop "
                 "create_channel create_nccl_group_channel create_nccl_group_channels create_channel_py_map "
                 "create_channel_py_single get_nccl_unique_id instantiate_channels init_engine init_engine_colocate "
                 "start_engine init_sampler init_tokenizer set_hosts").split()
    missing = [n for n in classes + functions if not hasattr(C, n)]
    assert not missing, missing
    x = torch.arange(12.0).view(4, 3)
    m = torch.tensor([3, 0, 2, 1, 7, 4, 6, 5])
    out = C.permute_tokens_cuda(x, m)
    for i in range(8):
        assert torch.equal(out[m[i]], x[i // 2])
