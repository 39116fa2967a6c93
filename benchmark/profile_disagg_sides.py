"""Stand-alone device time of each side of the fused disaggregated pipeline on ONE GPU (no peer has to exist):

  attention side   one iteration of an attention rank (2 micro-batches x all layers) with every flag pre-satisfied, so no
                   wait blocks and the dispatch stores land in a local arena
  expert side      one iteration of an expert rank holding `--experts-per-rank` experts per layer, fed with a fixed
                   number of rows per expert, arrival flags pre-satisfied

    python benchmark/profile_disagg_sides.py --n-attn 4 --n-expert 4

The two numbers bound the pipelined step time from below (the slower side) and from above (their sum).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from disagmoe_b200.config import get_preset
from disagmoe_b200.ops import _lib, gemm
from disagmoe_b200.parallel.disagg import AttentionRank, DisaggShape, ExpertRank, build_layout
from disagmoe_b200.parallel.peer import PeerArena


def timed(fn, iters=5, graph=True):
    """Median device time of fn(); with `graph` the launches are captured once and replayed, as the serving loop does
    (eager launches through ctypes cost more host time than the small attention-side kernels run)."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        fn = g.replay
        fn()
        torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def timeline(fn, per):
    """Per-kernel device time (us per layer and micro-batch for the per-layer kernels) of one eager run of fn()."""
    fn()
    torch.cuda.synchronize()
    _lib.start_timeline()
    fn()
    tl = _lib.stop_timeline()
    return ", ".join(f"{k} {ms * 1e3 / n:.1f} us x {n}" for k, (n, ms) in sorted(tl.items(), key=lambda kv: -kv[1][1]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--n-attn", type=int, default=4)
    ap.add_argument("--n-expert", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=864)
    ap.add_argument("--side", default="both")
    ap.add_argument("--timeline", action="store_true", help="also print the device time per kernel of one eager iteration "
                    "(a timing event after every launch; the GPU stays backlogged, so gaps between kernels are small)")
    ap.add_argument("--parts", action="store_true", help="attention side: also time a graph of each stage alone (norm + "
                    "all-gather push; QKV + attention + o_proj; reduce + router + dispatch) over all layers")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    ap.add_argument("--tp", type=int, default=1, help="attention tensor-parallel degree: the measured rank is member 0 of a "
                    "TP group that serves tp x batch rows (its peers' flags are pre-satisfied)")
    a = ap.parse_args()
    cfg = get_preset(a.model).clone(num_layers=a.layers)
    S = DisaggShape(a.n_attn, a.n_expert, 2, a.batch * a.tp, cfg.top_k, cfg.hidden_size, cfg.num_experts, a.tp)
    layout = build_layout(S)
    big = 2 ** 30
    if a.side in ("both", "attn"):
        arenas = PeerArena.emulated(a.n_attn + a.n_expert, layout.size)
        B = a.batch * a.tp
        blocks = 2 * B * ((a.ctx + 32) // 16 + 1) + 8
        r = AttentionRank(cfg, S, arenas[0], layout, 0, blocks)
        r.kv_cache.normal_(0, 0.5)
        per = (a.ctx + 32) // 16 + 1
        for m, d in enumerate(r.mb):
            d["comb_flag"].fill_(big)
            for k in ("hsflag", "oflag", "nidflag"):
                if k in d:
                    d[k].fill_(big)
            d["ids"].random_(0, cfg.vocab_size)
            d["positions"].fill_(a.ctx); d["ctx_len"].fill_(a.ctx + 1)
            rows = torch.arange(B, dtype=torch.int32, device="cuda") + m * B
            d["bt_row"].copy_(rows)
            bt = (rows.long()[:, None] * per + torch.arange(per, device="cuda")[None]).int()
            r.block_tables[m * B:(m + 1) * B, :per] = bt
            d["slots"].copy_(bt[:, a.ctx // 16].long() * 16 + a.ctx % 16)
        cursors = [arenas[a.n_attn + x].view(layout.offset(f"recv_cnt{m}"), (S.experts_per_rank,), torch.int32)
                   for x in range(a.n_expert) for m in range(2)]

        def attn_it():
            for m in range(2):
                r.embed(m)
            for l in range(cfg.num_layers):
                torch._foreach_zero_(cursors)      # no expert rank runs here to clear the row cursors it consumed
                for m in range(2):
                    r.layer(l, m)
            for m in range(2):
                r.head(m)
            for m in range(2):
                r.head_wait(m)
        ms = timed(attn_it, graph=not a.eager)
        print(f"attention side (tp {a.tp}, {B} rows per micro-batch): {ms:.2f} ms per iteration ({ms / a.layers / 2 * 1e3:.0f} us per layer and micro-batch), "
              f"status {gemm.check_status()}")
        if a.timeline:
            print("  per kernel:", timeline(attn_it, a.layers * 2))
        if a.parts:
            def stage(fn):
                def run():
                    for l in range(cfg.num_layers):
                        if fn == r.layer_route_dispatch:
                            torch._foreach_zero_(cursors)
                        for m in range(2):
                            fn(l, m)
                return timed(run, graph=True) / a.layers / 2 * 1e3
            one = lambda part: stage(lambda l, m: r.layer_attn(l, m, parts=(part,)))
            print(f"  stages alone, us per layer and micro-batch (graph replay): norm_gather {stage(r.layer_pre):.1f}, "
                  f"qkv {one('qkv'):.1f}, attention {one('attn'):.1f}, o_proj {one('o_proj'):.1f}, "
                  f"route_dispatch {stage(r.layer_route_dispatch):.1f}")
        del r, arenas
        torch.cuda.empty_cache()
    if a.side in ("both", "expert"):
        arenas = PeerArena.emulated(a.n_attn + a.n_expert, layout.size)
        x = ExpertRank(cfg, S, arenas[a.n_attn], layout, 0)
        pairs = a.n_attn * a.batch * cfg.top_k // cfg.num_experts      # rows per expert per launch (any TP degree)
        for d in x.mb:
            d["flag"].fill_(big)
            d["cnt"].fill_(pairs)
            d["rows"].normal_(0, 1)
            d["recs"].zero_()
            d["recs"][:, 1] = torch.arange(d["recs"].shape[0], device="cuda").int() % (a.batch * cfg.top_k)
        def it():
            for l in range(cfg.num_layers):
                for m in range(2):
                    x.layer(l, m)
                    x.mb[m]["cnt"].fill_(pairs)      # the combine cleared the cursors; refill for the next launch
        ms = timed(it, graph=not a.eager)
        print(f"expert side ({S.experts_per_rank} experts/GPU, {pairs} rows per expert, tile {x.bn}): {ms:.2f} ms per "
              f"iteration ({ms / a.layers / 2 * 1e3:.0f} us per layer and micro-batch), status {gemm.check_status()}")
        if a.timeline:
            print("  per kernel:", timeline(it, a.layers * 2))


if __name__ == "__main__":
    main()
