"""The colocated whole-iteration executor (CPU, fp32) against the independent fp32 oracle."""
import pytest
import torch

from disagmoe_b200.config import CacheConfig, tiny_config
from disagmoe_b200.executor.fused import FusedModelExecutor
from disagmoe_b200.models.oracle import OracleModel
from disagmoe_b200.models.weights import init_state_dict


def _run(cfg, prompts, n_new):
    sd = init_state_dict(cfg)
    oracle = OracleModel(cfg, sd)
    ex = FusedModelExecutor(cfg, CacheConfig(block_size=16), device="cpu", dtype=torch.float32, max_batch_size=8,
                            max_prefill_tokens=256, state_dict=sd, num_blocks=64, enable_cuda_graph=False)
    bs = 16
    # trivial block allocation: sequence r owns blocks [r * 8, r * 8 + 8)
    for r in range(len(prompts)):
        ex.set_block_table_row(r, list(range(r * 8, r * 8 + 8)))
    slot = lambda r, pos: (r * 8 + pos // bs) * bs + pos % bs
    ids, pos, slots, ctx, rows = [], [], [], [], []
    for r, p in enumerate(prompts):
        for i, t in enumerate(p):
            ids.append(t); pos.append(i); slots.append(slot(r, i)); ctx.append(i + 1); rows.append(r)
    ti = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt)
    _, logits = ex.prefill(ti(ids), ti(pos), ti(slots, torch.int64), ti(ctx), ti(rows), want_logits=True)
    ends = torch.tensor([len(p) for p in prompts]).cumsum(0) - 1
    cur = logits[ends].argmax(-1).tolist()
    ref_logits = [oracle.forward(r, p)[-1] for r, p in enumerate(prompts)]
    assert (logits[ends] - torch.stack(ref_logits)).abs().max() < 1e-4
    lens = [len(p) for p in prompts]
    for step in range(n_new):
        B = len(prompts)
        _, lg = ex.decode(ti(cur), ti(lens), ti([slot(r, lens[r]) for r in range(B)], torch.int64),
                          ti([l + 1 for l in lens]), ti(list(range(B))), want_logits=True)
        ref = torch.stack([oracle.forward(r, [cur[r]])[-1] for r in range(B)])
        assert (lg - ref).abs().max() < 1e-4, f"decode step {step}"
        cur = lg.argmax(-1).tolist()
        lens = [l + 1 for l in lens]


def test_tiny_mixtral_matches_oracle():
    torch.manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,)).tolist() for n in (32, 7, 19)]
    _run(tiny_config, prompts, 4)


def test_shared_expert_and_dense_layer_match_oracle():
    cfg = tiny_config.clone(num_layers=3, first_k_dense=1, dense_intermediate_size=384, num_shared_experts=1,
                            shared_intermediate_size=256, shared_expert_gate=True, norm_topk_prob=False, top_k=3,
                            num_kv_heads=2)
    torch.manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,)).tolist() for n in (9, 21)]
    _run(cfg, prompts, 3)


def test_trace_weighted_router_file(tmp_path, monkeypatch):
    """DMOE_WEIGHTED_ROUTER_FILE: per-layer expert popularity from a routing-trace CSV; the router then samples expert
    ids from it, or (use_popularity_as_logit_bias) keeps the gate and skews its logits."""
    import pandas as pd
    import torch
    from disagmoe_b200.config import tiny_config
    from disagmoe_b200.models.attention import MoEAttention
    E = tiny_config.num_experts
    rows = []
    for layer in range(2):
        for cat in ("closed_qa", "other"):
            for _ in range(3):
                counts = [0] * E
                counts[layer] = 90 if cat == "closed_qa" else 1         # layer l prefers expert l
                counts[E - 1] = 10
                rows.append({"category": cat, "layer_id": layer, **{f"e{i}": c for i, c in enumerate(counts)}})
    path = tmp_path / "trace.csv"
    pd.DataFrame(rows).to_csv(path, index=False)
    monkeypatch.setenv("DMOE_WEIGHTED_ROUTER_FILE", str(path))
    a = MoEAttention(tiny_config, 1)
    a.init_weights()
    assert torch.allclose(a.weighted_router, torch.tensor([0, 0.9, 0, 0, 0, 0, 0, 0.1]), atol=1e-6)
    x = torch.randn(200, tiny_config.hidden_size)
    _, ids, w, _ = a.route(x)
    assert set(ids.reshape(-1).tolist()) == {1, E - 1}                 # only experts with non-zero popularity
    assert torch.allclose(w.sum(1), torch.ones(200))
    a.use_popularity_as_logit_bias()
    assert a.weighted_router is None and a.route_bias.argmax().item() == 1
    _, ids, _, _ = a.route(x)
    hist = torch.bincount(ids.reshape(-1).long(), minlength=E)
    assert hist[1] >= 190 and hist[E - 1] >= 150                       # the gate decides, heavily skewed
    monkeypatch.delenv("DMOE_WEIGHTED_ROUTER_FILE")
    assert MoEAttention(tiny_config, 1).weighted_router is None


def test_expert_shard_init_equals_slices_of_the_full_state_dict():
    """An expert-parallel worker started without a state dict draws only its own experts; they must be the
    transposed slices of the tensors a single-process model (or the oracle) is initialised with."""
    import torch
    from disagmoe_b200.config import tiny_config
    from disagmoe_b200.models import weights as W
    from disagmoe_b200.models.experts import MoEExperts
    cfg = tiny_config.clone(dtype=torch.float32)
    sd = W.init_state_dict(cfg)
    for lo, hi in [(0, cfg.num_experts), (2, 5)]:
        a = MoEExperts(cfg, 1, lo, hi)
        a.init_weights()
        b = MoEExperts(cfg, 1, lo, hi)
        b.load_weights(sd)
        assert torch.equal(a.w13_weight, b.w13_weight) and torch.equal(a.w2_weight, b.w2_weight)
