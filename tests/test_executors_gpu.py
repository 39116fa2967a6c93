"""Per-layer executors on the GPU: eager vs CUDA-graph attention executor, grouped vs serial experts executor."""
import pytest
import torch

from disagmoe_b200.config import CacheConfig, tiny_config
from disagmoe_b200.executor.executor import AttnExecutor, CUDAGraphAttnExecutor, ExpertsExecutor
from disagmoe_b200.models.attention import AttnMeta
from disagmoe_b200.models.weights import init_state_dict

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    return tiny_config.clone(dtype=torch.bfloat16, max_batch_size_attn=16, graph_stride=8, max_seq_len=256, **kw)


def test_cuda_graph_attention_executor_matches_eager():
    cfg = _cfg()
    sd = {k: v.to(torch.bfloat16) for k, v in init_state_dict(cfg, dtype=torch.float32).items()}
    cc = CacheConfig(block_size=16)
    eager = AttnExecutor(cfg, cc, state_dict=sd)
    graphed = AttnExecutor(cfg, cc, state_dict=sd)
    eager.initialize_cache(32)
    graphed.initialize_cache(32)
    g = torch.Generator().manual_seed(0)
    kv = (torch.randn(eager.cache.shape, generator=g) * 0.5).to(torch.bfloat16).cuda()
    eager.cache.copy_(kv)
    graphed.cache.copy_(kv)
    cg = CUDAGraphAttnExecutor(cfg, cc, graphed)
    cg.create_cuda_graph_buffers()
    assert cg.graph_batch_sizes == [1, 8, 16]
    cg.capture()
    graphed.cache.copy_(kv)          # capture warm-ups appended nothing (slots = -1), but keep the caches identical
    n = 5
    x = torch.randn(n, cfg.hidden_size, generator=g).to(torch.bfloat16).cuda()
    ctx = torch.tensor([3, 17, 30, 9, 22], dtype=torch.int32, device="cuda")
    bt = torch.arange(n * 2, dtype=torch.int32, device="cuda").view(n, 2)
    slots = (bt.gather(1, (ctx // 16).long()[:, None]).squeeze(1).long() * 16 + (ctx % 16).long())
    meta = AttnMeta(ctx.clone(), slots, bt, None, ctx + 1, num_decode_tokens=n, max_ctx=64)
    for layer in (0, 1):
        xe = x.clone()
        ye, we, ie = eager.execute(layer, ctx, xe, meta)
        yg, wg, ig, xg = cg.run(layer, ctx, x.clone(), meta)
        torch.cuda.synchronize()
        assert torch.equal(ie, ig) and torch.allclose(we, wg) and torch.equal(ye, yg) and torch.equal(xe, xg)


def test_experts_executor_grouped_equals_serial():
    cfg = _cfg(ep_size=2)
    sd = {k: v.to(torch.bfloat16) for k, v in init_state_dict(cfg, dtype=torch.float32).items()}
    grouped = ExpertsExecutor(cfg, state_dict=sd, e_lo=4)
    serial = ExpertsExecutor(cfg.clone(enable_grouped_gemm=False), state_dict=sd, e_lo=4)
    assert grouped.operators[0].num_experts == 4
    sizes = torch.tensor([5, 0, 9, 2])
    x = torch.randn(int(sizes.sum()), cfg.hidden_size).to(torch.bfloat16).cuda()
    a = grouped.execute(1, x.shape[0], x, sizes).clone()
    b = serial.execute(1, x.shape[0], x, sizes)
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max() / b.float().abs().max() < 2e-2
