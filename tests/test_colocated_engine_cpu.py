"""The single-device serving engine (CPU, fp32): continuous batching + native block manager vs the oracle."""
import torch

from disagmoe_b200.config import CacheConfig, tiny_config
from disagmoe_b200.frontend.colocated import ColocatedEngine
from disagmoe_b200.models.oracle import OracleModel
from disagmoe_b200.models.weights import init_state_dict


def test_engine_generates_oracle_tokens():
    cfg = tiny_config
    sd = init_state_dict(cfg)
    eng = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cpu", max_batch_size=4, max_prefill_tokens=64,
                          state_dict=sd, num_blocks=64, enable_cuda_graph=False, dtype=torch.float32)
    torch.manual_seed(0)
    prompts = {i: torch.randint(0, cfg.vocab_size, (n,)).tolist() for i, n in enumerate((32, 5, 17, 30, 9, 12))}
    new = {0: 6, 1: 3, 2: 18, 3: 5, 4: 7, 5: 4}     # request 2 crosses a block boundary while decoding
    for i, p in prompts.items():
        eng.add_request(i, p, new[i])
    out = eng.run_until_done(max_steps=200)
    assert not eng.has_unfinished()
    oracle = OracleModel(cfg, sd)
    for i, p in prompts.items():
        ref, _ = oracle.generate(i, p, new[i])
        assert out[i] == ref, f"request {i}"
    # every KV block went back to the allocator
    assert eng.block_mgr.num_free_blocks() == 64 and eng.block_mgr.num_seqs() == 0


def test_tight_kv_pool_admission_waits_instead_of_failing():
    """More requests than the KV pool can hold at once: admission reserves the blocks running sequences will grow into,
    so the engine works through the queue without ever running out of blocks."""
    import torch
    from disagmoe_b200.config import CacheConfig, tiny_config
    from disagmoe_b200.frontend.colocated import ColocatedEngine
    cfg = tiny_config.clone(dtype=torch.float32, num_layers=1)
    eng = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cpu", max_batch_size=8, max_prefill_tokens=128,
                          num_blocks=14, enable_cuda_graph=False)
    g = torch.Generator().manual_seed(0)
    for i in range(10):
        n = int(torch.randint(5, 40, (1,), generator=g))
        eng.add_request(i, torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), 30)
    out = eng.run_until_done(5000)
    assert len(out) == 10 and all(len(v) == 30 for v in out.values())


def test_mixed_batch_engine_matches_alternating_engine():
    """Mixed batches with chunked prefill (prompt budget 16 rows per step, prompts up to 45 tokens) produce the same
    greedy tokens as the engine that prefills whole prompts in steps of their own."""
    import torch
    from disagmoe_b200.config import CacheConfig, tiny_config
    from disagmoe_b200.frontend.colocated import ColocatedEngine
    from disagmoe_b200.frontend.colocated_mixed import MixedBatchEngine
    from disagmoe_b200.models.weights import init_state_dict
    cfg = tiny_config.clone(dtype=torch.float32)
    sd = init_state_dict(cfg)
    g = torch.Generator().manual_seed(4)
    reqs = [(i, torch.randint(0, cfg.vocab_size, (int(torch.randint(3, 46, (1,), generator=g)),), generator=g).tolist(),
             int(torch.randint(2, 9, (1,), generator=g))) for i in range(9)]
    kw = dict(device="cpu", max_batch_size=4, max_prefill_tokens=64, num_blocks=96, enable_cuda_graph=False, state_dict=sd)
    a = ColocatedEngine(cfg, CacheConfig(block_size=16), **kw)
    b = MixedBatchEngine(cfg, CacheConfig(block_size=16), prefill_budget=16, **kw)
    for rid, prompt, n_out in reqs:
        a.add_request(rid, prompt, n_out)
        b.add_request(rid, prompt, n_out)
    want = a.run_until_done(2000)
    steps = 0
    saw_mixed = False
    while b.has_unfinished():
        before = {r for r in b.sched.running[0]}
        out = b.step()
        saw_mixed |= bool(before) and any(s.length < len(s.prompt) for s in b.sched.running[0].values())
        steps += 1
        assert steps < 2000
    got = {r: s.outputs for r, s in b.finished.items()}
    assert got == want
    assert saw_mixed, "the workload was meant to overlap a chunked prompt with running sequences"
    assert b.block_mgr.num_free_blocks() == a.block_mgr.num_free_blocks()


def test_mixed_batch_engine_snapshot_resumes_with_identical_tokens(tmp_path):
    """Snapshot in the middle of a chunked prefill and of decoding sequences; a fresh engine continues identically."""
    import torch
    from disagmoe_b200.config import CacheConfig, tiny_config
    from disagmoe_b200.frontend.colocated_mixed import MixedBatchEngine
    from disagmoe_b200.models.weights import init_state_dict
    cfg = tiny_config.clone(dtype=torch.float32)
    sd = init_state_dict(cfg)
    g = torch.Generator().manual_seed(9)
    reqs = [(i, torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), 7) for i, n in enumerate([6, 50, 9, 44])]
    kw = dict(device="cpu", max_batch_size=4, max_prefill_tokens=64, num_blocks=96, enable_cuda_graph=False, state_dict=sd,
              prefill_budget=16)
    ref = MixedBatchEngine(cfg, CacheConfig(block_size=16), **kw)
    a = MixedBatchEngine(cfg, CacheConfig(block_size=16), **kw)
    for r in reqs:
        ref.add_request(*r)
        a.add_request(*r)
    want = ref.run_until_done(500)
    for _ in range(3):
        a.step()
    assert any(s.length < len(s.prompt) for s in a.sched.running[0].values()), "a prompt should be part-way through"
    path = str(tmp_path / "state.pt")
    a.save_state(path)
    b = MixedBatchEngine(cfg, CacheConfig(block_size=16), **kw)
    b.load_state(path)
    assert b.run_until_done(500) == want
