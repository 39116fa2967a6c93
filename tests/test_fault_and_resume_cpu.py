"""Failure detection, checkpoint layout / sharding, and serving-state resume -- all on CPU, no device is ever faulted:
a failure is a worker process that exits between steps, seen by the controller through process liveness."""
import os
import tempfile
import time

import pytest
import torch

from disagmoe_b200.config import CacheConfig, SamplingConfig, mixtral_config, tiny_config
from disagmoe_b200.frontend.colocated import ColocatedEngine
from disagmoe_b200.frontend.controller import init_controller
from disagmoe_b200.models import weights as W
from disagmoe_b200.models.linear import QKVParallelLinear, RowParallelLinear
from disagmoe_b200.utils.placement import ClusterConfig, get_model_placement


def test_dead_worker_is_detected_and_requests_fail_fast():
    cfg = tiny_config.clone(ep_size=1)
    place = get_model_placement(cfg, ClusterConfig(1, 2), "pipeline", 1, 1)
    ctl = init_controller(1, 2, device="cpu")
    try:
        ctl.init_engine(place, cfg, CacheConfig(block_size=16, num_gpu_blocks=64), SamplingConfig(2, 3),
                        dtype=torch.float32)
        ctl.start_engine()
        r = ctl.put_single_request([5, 6, 7], output_len=2)
        r.get(timeout=60)                       # the system works
        assert ctl.check_workers() == []
        # the expert worker leaves between steps (nothing in flight); the controller learns it on the host
        ctl.workers[1].proc.terminate()
        ctl.workers[1].proc.join(timeout=10)
        assert ctl.check_workers() == [1] and ctl.suspect_workers == [1]
        ctl.put_single_request([8, 9, 10], output_len=2)
        t0 = time.time()
        with pytest.raises(RuntimeError, match="worker 1 died"):
            ctl.wait_for_requests(2, timeout=30)
        assert time.time() - t0 < 5, "a dead peer must surface quickly, not after the request timeout"
    finally:
        ctl.stop_workers()


def test_state_dict_save_load_and_sharding_rules():
    cfg = tiny_config.clone(num_kv_heads=2)
    sd = W.init_state_dict(cfg)
    assert W.check_state_dict(cfg, sd) == []
    path = os.path.join(tempfile.mkdtemp(), "ckpt.pt")
    W.save_state_dict(sd, path)
    back = W.load_state_dict(path)
    assert all(torch.equal(sd[k], back[k]) for k in sd)
    # seeded init is independent of which tensors a process materialises
    one = W.init_state_dict(cfg, names=["layers.1.gate.weight"])
    assert torch.equal(one["layers.1.gate.weight"], sd["layers.1.gate.weight"])
    # TP shards: the functional rule and the layer's weight_loader agree (kv heads replicated when tp > kv heads)
    full = sd["layers.0.qkv_proj.weight"]
    for tp in (2, 4):
        for r in range(tp):
            lin = QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, tp_size=tp, tp_rank=r,
                                    params_dtype=torch.float32)
            lin.weight_loader(lin.weight, full)
            assert torch.equal(lin.weight.data, W.shard_qkv(full, cfg, tp, r))
            o = RowParallelLinear(cfg.num_heads * cfg.head_dim, cfg.hidden_size, tp_size=tp, tp_rank=r,
                                  params_dtype=torch.float32)
            o.weight_loader(o.weight, sd["layers.0.o_proj.weight"])
            assert torch.equal(o.weight.data, W.shard_o_proj(sd["layers.0.o_proj.weight"], cfg, tp, r))
    # expert slices and the runtime (K-contiguous) layout round trip
    w13, w2 = sd["layers.0.experts.w13_weight"], sd["layers.0.experts.w2_weight"]
    r13, r2 = W.to_runtime_expert_layout(W.shard_experts(w13, 2, 4), W.shard_experts(w2, 2, 4))
    assert r13.shape == (2, 2 * cfg.intermediate_size, cfg.hidden_size) and r2.shape == (2, cfg.hidden_size, cfg.intermediate_size)
    c13, c2 = W.to_checkpoint_expert_layout(r13, r2)
    assert torch.equal(c13, w13[2:4]) and torch.equal(c2, w2[2:4])
    shapes = W.param_shapes(mixtral_config)
    assert shapes["layers.0.qkv_proj.weight"] == (6144, 4096) and shapes["layers.31.experts.w13_weight"] == (8, 4096, 28672)


def test_serving_state_snapshot_resumes_with_identical_tokens():
    cfg = tiny_config
    sd = W.init_state_dict(cfg)
    mk = lambda: ColocatedEngine(cfg, CacheConfig(block_size=16), device="cpu", max_batch_size=4, max_prefill_tokens=64,
                                 state_dict=sd, num_blocks=64, enable_cuda_graph=False, dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    prompts = {i: torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for i, n in enumerate((14, 30, 9))}
    ref = mk()
    for i, p in prompts.items():
        ref.add_request(i, p, 12)
    want = ref.run_until_done(100)
    a = mk()
    for i, p in prompts.items():
        a.add_request(i, p, 12)
    for _ in range(5):
        a.step()
    path = os.path.join(tempfile.mkdtemp(), "serving_state.pt")
    a.save_state(path)
    del a
    b = mk()
    # occupy some blocks first so that the restored sequences land on different physical pages
    b.block_mgr.allocate(999, 40); b.block_mgr.drain_updates()
    b.load_state(path)
    got = b.run_until_done(100)
    assert got == want


def test_recover_restarts_workers_and_readmits_unfinished_requests():
    """The expert worker process dies while requests are decoding. ``Controller.recover`` rebuilds every worker and
    re-admits the unfinished requests as prompt + tokens produced so far; the final token lists equal the oracle's."""
    import os
    import tempfile
    from disagmoe_b200.models.oracle import OracleModel
    from disagmoe_b200.models.weights import init_state_dict, save_state_dict
    cfg = tiny_config.clone(ep_size=1)
    sd = init_state_dict(cfg)
    path = os.path.join(tempfile.mkdtemp(), "tiny.pt")
    save_state_dict(sd, path)
    place = get_model_placement(cfg, ClusterConfig(1, 2), "pipeline", 1, 1)
    ctl = init_controller(1, 2, device="cpu")
    n_new = 40
    try:
        ctl.init_engine(place, cfg, CacheConfig(block_size=16, num_gpu_blocks=128), SamplingConfig(n_new, n_new + 1),
                        state_dict_path=path, dtype=torch.float32)
        ctl.start_engine()
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(3, cfg.vocab_size, (10,), generator=g).tolist() for _ in range(4)]
        res = [ctl.put_single_request(p, output_len=n_new) for p in prompts]
        t0 = time.time()
        while len(ctl.sampler.get_output_tokens(res[0].req_id)) < 3:
            assert time.time() - t0 < 60
            time.sleep(0.001)
        ctl.workers[1].proc.terminate()           # between two of its steps as far as the GPU-less worker is concerned
        ctl.workers[1].proc.join(timeout=10)
        assert ctl.check_workers() == [1]
        again = ctl.recover()
        assert again, "the worker died before the requests had finished, so some must be re-admitted"
        assert ctl.check_workers() == []
        ctl.wait_for_requests(4, timeout=120)
        oracle = OracleModel(cfg, sd)
        for r, p in zip(res, prompts):
            want, _ = oracle.generate(r.req_id, p, n_new)
            assert r.tokens == want, f"request {r.req_id}"
    finally:
        ctl.stop_workers()


def _tiny_job(n_new, **init_kw):
    import os
    import tempfile
    from disagmoe_b200.models.oracle import OracleModel
    from disagmoe_b200.models.weights import init_state_dict, save_state_dict
    cfg = tiny_config.clone(ep_size=1)
    sd = init_state_dict(cfg)
    path = os.path.join(tempfile.mkdtemp(), "tiny.pt")
    save_state_dict(sd, path)
    place = get_model_placement(cfg, ClusterConfig(1, 2), "pipeline", 1, 1)
    ctl = init_controller(1, 2, device="cpu", in_process=True)
    ctl.init_engine(place, cfg, CacheConfig(block_size=16, num_gpu_blocks=128), SamplingConfig(n_new, n_new + 1),
                    state_dict_path=path, dtype=torch.float32)
    ctl.start_engine()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, cfg.vocab_size, (9,), generator=g).tolist() for _ in range(3)]
    return cfg, ctl, prompts, OracleModel(cfg, sd)


@pytest.mark.parametrize("kind", ["duplicate", "delay"])
def test_duplicated_or_delayed_message_does_not_change_the_result(kind):
    """Host-side fault hook on the message layer: one message is sent twice (the receiver's sequence filter drops the
    copy) or held back for 150 ms. The generated tokens still equal the oracle's."""
    from disagmoe_b200 import disagmoe_c as C
    n_new = 6
    cfg, ctl, prompts, oracle = _tiny_job(n_new)
    try:
        fired0 = C.send_faults_fired()
        C.set_send_fault(C.SEND_FAULT_DUPLICATE if kind == "duplicate" else C.SEND_FAULT_DELAY, 7, 150)
        res = [ctl.put_single_request(p, output_len=n_new) for p in prompts]
        ctl.wait_for_requests(3, timeout=120)
        assert C.send_faults_fired() == fired0 + 1
        for r, p in zip(res, prompts):
            assert r.tokens == oracle.generate(r.req_id, p, n_new)[0]
        assert not [e for e in ctl.worker_errors().values() if e]
    finally:
        ctl.stop_workers()


def test_dropped_message_is_noticed_by_the_deadline_and_recovered():
    """One message is dropped on the host: the tokens it carried never arrive, the affected requests stop making
    progress. The controller's per-request deadline reports them and recover() finishes every request."""
    from disagmoe_b200 import disagmoe_c as C
    n_new = 8
    cfg, ctl, prompts, oracle = _tiny_job(n_new)
    try:
        C.set_send_fault(C.SEND_FAULT_DROP, 9)
        res = [ctl.put_single_request(p, output_len=n_new) for p in prompts]
        t0 = time.time()
        while not ctl.stalled_requests(0.5):
            assert time.time() - t0 < 30, "the stall was not reported"
            time.sleep(0.05)
        stalled = ctl.stalled_requests(0.5)
        assert set(stalled) <= {r.req_id for r in res}
        ctl.recover()
        ctl.wait_for_requests(3, timeout=120)
        for r, p in zip(res, prompts):
            assert r.tokens == oracle.generate(r.req_id, p, n_new)[0]
    finally:
        ctl.stop_workers()
