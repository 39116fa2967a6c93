"""The correctness line of ``bench.py`` (tiny 2-layer MoE through the fused pipeline vs the colocated executor) for a
tensor-parallel attention group of ``tp`` GPUs + 4 expert GPUs, emulated on ONE GPU: every rank's kernels run on the
same device over arenas that address each other, phase by phase, so no kernel ever waits and no race is possible.

    python benchmark/emulated_selfcheck.py [tp]        # default 4: the 8-GPU layout

Prints the per-row error of every rank. The inputs, seeds and weights are those of the multi-GPU selfcheck
(``parallel/disagg.py: selfcheck_against_colocated``), so a multi-GPU run that reports the same numbers computed
exactly what this sequential run computes: what differs from the colocated logits is then arithmetic (the bf16
summation order of the o_proj partial sums, which can flip a router near-tie), not ordering between GPUs."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from disagmoe_b200.config import CacheConfig, tiny_config
from disagmoe_b200.executor.fused import FusedModelExecutor
from disagmoe_b200.models import weights as W
from disagmoe_b200.ops import gemm
from disagmoe_b200.parallel.disagg import AttentionRank, DisaggShape, ExpertRank, build_layout, shard_rows
from disagmoe_b200.parallel.peer import PeerArena


def main(tp: int = 4, n_expert: int = 4, n_mb: int = 2, batch: int = 8) -> None:
    A, X = tp, n_expert
    cfg = tiny_config.clone(dtype=torch.bfloat16, num_layers=2)
    sd = {k: v.to(torch.bfloat16) for k, v in W.init_state_dict(cfg, dtype=torch.float32).items()}
    B = batch * tp
    shape = DisaggShape(A, X, n_mb, B, cfg.top_k, cfg.hidden_size, cfg.num_experts, tp)
    layout = build_layout(shape)
    arenas = PeerArena.emulated(A + X, layout.size)
    nb, bs = 4 * n_mb * B + 1, 16
    attn = [AttentionRank(cfg, shape, arenas[a], layout, a, nb, state_dict=sd) for a in range(A)]
    exps = [ExpertRank(cfg, shape, arenas[A + x], layout, x, state_dict=sd) for x in range(X)]
    kvh = cfg.num_kv_heads // tp
    # every member of the group draws the same KV history and requests (generator seed of group 0 in the selfcheck)
    g = torch.Generator().manual_seed(99)
    kv = torch.randn(cfg.num_layers, 2, nb, bs, cfg.num_kv_heads, cfg.head_dim, generator=g).to(torch.bfloat16) * 0.5
    inputs = []
    for m in range(n_mb):
        ids = torch.randint(0, cfg.vocab_size, (B,), generator=g).int()
        ctx = torch.randint(3, 60, (B,), generator=g).int()
        bt = (torch.arange(B * 4, dtype=torch.int32) + m * B * 4).view(B, 4)
        slots = torch.tensor([int(bt[i, int(ctx[i]) // bs]) * bs + int(ctx[i]) % bs for i in range(B)])
        inputs.append((ids, ctx, slots, bt))
    for rank, r in enumerate(attn):
        r.kv_cache.copy_(kv[..., rank * kvh:(rank + 1) * kvh, :])
        for m, (ids, ctx, slots, bt) in enumerate(inputs):
            r.block_tables[m * B:(m + 1) * B, :4] = bt.cuda()
            d = r.mb[m]
            d["ids"].copy_(ids); d["positions"].copy_(ctx); d["ctx_len"].copy_(ctx + 1)
            d["bt_row"].copy_(torch.arange(B, dtype=torch.int32) + m * B); d["slots"].copy_(slots)
    # one stream, several ranks: every phase is launched for all ranks before the phase that waits for it
    for a in attn:
        for m in range(n_mb):
            a.embed(m)
    for l in range(cfg.num_layers):
        for m in range(n_mb):
            for a in attn:
                a.layer_pre(l, m)
            for a in attn:
                a.layer_attn(l, m)
            for a in attn:
                a.layer_route_dispatch(l, m)
            for e in exps:
                e.layer(l, m)
    for a in attn:
        for m in range(n_mb):
            a.head(m)
    for a in attn:
        for m in range(n_mb):
            a.head_wait(m)
    torch.cuda.synchronize()
    print("kernel status", gemm.check_status())
    ref = FusedModelExecutor(cfg, CacheConfig(block_size=bs), device="cuda", max_batch_size=B, max_prefill_tokens=B,
                             state_dict=sd, num_blocks=nb, enable_cuda_graph=False)
    per = shard_rows(B, tp)
    worst, agree_min = 0.0, 1.0
    for m, (ids, ctx, slots, bt) in enumerate(inputs):
        ref.kv_cache.copy_(kv.cuda())
        ref.block_tables[:B, :4] = bt.cuda()
        _, lg = ref.decode(ids, ctx, slots, ctx + 1, torch.arange(B, dtype=torch.int32), want_logits=True)
        for ri, r in enumerate(attn):
            lo, hi = min(B, ri * per), min(B, (ri + 1) * per)
            got, want = r.mb[m]["logits"][:hi - lo].float(), lg[lo:hi].float()
            row_err = (got - want).abs().amax(-1) / want.abs().max()
            ag = (got.argmax(-1) == want.argmax(-1)).float()
            worst, agree_min = max(worst, float(row_err.max())), min(agree_min, float(ag.mean()))
            print(f"micro-batch {m} rank {ri}: row errors {[round(float(x), 4) for x in row_err]} "
                  f"arg-max agrees {[int(x) for x in ag]}")
    print("max_rel_err", round(worst, 6), "argmax_agree_min", agree_min)


if __name__ == "__main__":
    main(int(sys.argv[1]) if len(sys.argv) > 1 else 4)
