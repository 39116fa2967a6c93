"""The colocated engine on the GPU (bf16 kernels, CUDA graph) against the fp32 oracle."""
import pytest
import torch

from disagmoe_b200.config import CacheConfig, tiny_config
from disagmoe_b200.frontend.colocated import ColocatedEngine
from disagmoe_b200.models.oracle import OracleModel
from disagmoe_b200.models.weights import init_state_dict
from disagmoe_b200.ops import gemm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["mixtral", "shared_dense"])
def test_gpu_engine_tracks_oracle(variant):
    cfg = tiny_config.clone(dtype=torch.bfloat16)
    if variant == "shared_dense":
        cfg = cfg.clone(num_layers=3, first_k_dense=1, dense_intermediate_size=384, num_shared_experts=1,
                        shared_intermediate_size=256, shared_expert_gate=True, norm_topk_prob=False, top_k=3,
                        num_kv_heads=2)
    sd = init_state_dict(cfg, dtype=torch.float32)
    sd_bf = {k: v.to(torch.bfloat16) for k, v in sd.items()}
    eng = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=8, max_prefill_tokens=128,
                          state_dict=sd_bf, num_blocks=64, enable_cuda_graph=True)
    eng.executor.capture([4, 8])
    oracle = OracleModel(cfg, {k: v.float() for k, v in sd_bf.items()})
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (32, 7, 19)]
    # teacher-forced comparison of logits: prefill, then 3 decode steps fed with the oracle's tokens
    ex = eng.executor
    for r in range(3):
        eng.block_mgr.allocate(r, 64)
    eng._apply_block_table_patches()
    ids, pos, slots, ctx, rows = [], [], [], [], []
    for r, p in enumerate(prompts):
        for i, t in enumerate(p):
            ids.append(t); pos.append(i); slots.append(eng.block_mgr.slot_of(r, i)); ctx.append(i + 1)
            rows.append(eng.block_mgr.row_of(r))
    ti = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt)
    _, logits = ex.prefill(ti(ids), ti(pos), ti(slots, torch.int64), ti(ctx), ti(rows), want_logits=True)
    ends = torch.tensor([len(p) for p in prompts]).cumsum(0) - 1
    ref = torch.stack([oracle.forward(r, p)[-1] for r, p in enumerate(prompts)])
    got = logits[ends.cuda()].float().cpu()
    scale = ref.abs().max()
    assert (got - ref).abs().max() / scale < 0.06
    assert (got.argmax(-1) == ref.argmax(-1)).float().mean() >= 2 / 3
    cur = ref.argmax(-1).tolist()
    lens = [len(p) for p in prompts]
    for step in range(3):
        B = 3
        _, lg = ex.decode(ti(cur), ti(lens), ti([eng.block_mgr.slot_of(r, lens[r]) for r in range(B)], torch.int64),
                          ti([l + 1 for l in lens]), ti([eng.block_mgr.row_of(r) for r in range(B)]), want_logits=True)
        ref = torch.stack([oracle.forward(r, [cur[r]])[-1] for r in range(B)])
        assert (lg.float().cpu() - ref).abs().max() / ref.abs().max() < 0.06, f"step {step}"
        cur = ref.argmax(-1).tolist()
        lens = [l + 1 for l in lens]
    torch.cuda.synchronize()
    assert gemm.check_status() == 0


def test_graph_replay_equals_eager():
    cfg = tiny_config.clone(dtype=torch.bfloat16)
    eng = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=8, max_prefill_tokens=64,
                          num_blocks=64, enable_cuda_graph=True)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 14, 5)]
    for i, p in enumerate(prompts):
        eng.add_request(i, p, 6)
    eager = eng.run_until_done(64)
    eng2 = ColocatedEngine(cfg, CacheConfig(block_size=16), device="cuda", max_batch_size=8, max_prefill_tokens=64,
                           num_blocks=64, enable_cuda_graph=True)
    eng2.executor.capture([4, 8])
    for i, p in enumerate(prompts):
        eng2.add_request(i, p, 6)
    graphed = eng2.run_until_done(64)
    assert eager == graphed
