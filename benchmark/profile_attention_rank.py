"""The fused attention-side and expert-side kernels of the disaggregated pipeline on ONE GPU, for per-kernel profiling.

    python benchmark/profile_attention_rank.py --tp 4 --experts-gpus 4 --batch 256 --layers 2 --steps 3

A whole job (``--tp`` attention ranks forming one tensor-parallel group + ``--experts-gpus`` expert ranks, Mixtral layer
shapes) is emulated on one device: every rank gets its own arena, the arenas simply address each other, and the
phases of a layer are launched for all ranks in an order in which no flag wait has to block (all ``norm_gather``, then
all QKV / attention / o_proj, then all ``route_dispatch``, then the experts). Kernel arguments, grids and memory
traffic per launch are those of the multi-GPU run, except that "peer" stores land in local memory. This is the
program to put under ``ncu -k regex:<kernel>``; a profiler must never wrap the multi-process run itself.
Prints the mean device time of one emulated iteration (all ranks back to back, so not a throughput number).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from disagmoe_b200.config import get_preset
from disagmoe_b200.ops import gemm
from disagmoe_b200.parallel.disagg import AttentionRank, DisaggShape, ExpertRank, build_layout
from disagmoe_b200.parallel.peer import PeerArena


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--tp", type=int, default=4)
    ap.add_argument("--experts-gpus", type=int, default=4)
    ap.add_argument("--batch", type=int, default=256, help="sequences per attention GPU (the group serves tp x batch rows)")
    ap.add_argument("--ctx", type=int, default=864)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    cfg = get_preset(args.model).clone(num_layers=args.layers, max_seq_len=4096)
    A, X, tp = args.tp, args.experts_gpus, args.tp
    B = args.batch * tp
    shape = DisaggShape(A, X, 1, B, cfg.top_k, cfg.hidden_size, cfg.num_experts, tp)
    layout = build_layout(shape)
    arenas = PeerArena.emulated(A + X, layout.size)
    blocks = B * ((args.ctx + args.steps + 17) // 16) + 8
    attn = [AttentionRank(cfg, shape, arenas[a], layout, a, num_blocks=blocks) for a in range(A)]
    exps = [ExpertRank(cfg, shape, arenas[A + x], layout, x) for x in range(X)]
    g = torch.Generator().manual_seed(0)
    per_seq = (args.ctx + args.steps + 17) // 16
    for a in attn:
        a.kv_cache.normal_(0, 0.5)
        bt = torch.arange(B * per_seq, dtype=torch.int32).view(B, per_seq)
        a.block_tables[:B, :per_seq] = bt.cuda()
        d = a.mb[0]
        d["ids"].copy_(torch.randint(0, cfg.vocab_size, (B,), generator=torch.Generator().manual_seed(1)).int())
        d["bt_row"].copy_(torch.arange(B, dtype=torch.int32))

    def iteration(step):
        pos = args.ctx + step
        for a in attn:
            d = a.mb[0]
            d["positions"].fill_(pos)
            d["ctx_len"].fill_(pos + 1)
            d["slots"].copy_((torch.arange(B) * per_seq * 16 + pos).long())
            a.embed(0)
        for l in range(cfg.num_layers):
            for a in attn:
                a.layer_pre(l, 0)
            for a in attn:
                a.layer_attn(l, 0)
            for a in attn:
                a.layer_route_dispatch(l, 0)
            for e in exps:
                e.layer(l, 0)
        for a in attn:
            a.head(0)
        for a in attn:
            a.head_wait(0)

    ms = []
    for step in range(args.steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        iteration(step)
        e.record()
        torch.cuda.synchronize()
        ms.append(round(s.elapsed_time(e), 2))
    print(f"model={cfg.name} layers={args.layers} tp={tp} expert_gpus={X} rows={B} ctx={args.ctx} "
          f"ms per emulated iteration={ms} kernel_status={gemm.check_status()}")


if __name__ == "__main__":
    main()
