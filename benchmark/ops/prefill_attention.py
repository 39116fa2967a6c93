"""Prompt (prefill) attention: the tiled causal kernel against the per-token paged kernel it replaces for prompt rows.

    python benchmark/ops/prefill_attention.py [--lens 128,512,1024,2048] [--seqs 4] [--heads 32 --kv-heads 8 --head-dim 128]

One batch of ``--seqs`` whole prompts of each length (K / V already appended to the paged cache, block size 16), CUDA-event
timing, median of ``--iters`` with a 256 MB buffer written between iterations. Prints both times, the K / V bytes each
kernel has to stream (the per-token kernel reads every row's own prefix; the tiled kernel reads the prefix once per tile
of 64 / (heads per kv head) tokens) and the ratio.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from disagmoe_b200.ops import functional as F


def timed(fn, flush, iters):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2] * 1e3


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--lens", default="128,512,1024,2048")
    ap.add_argument("--seqs", type=int, default=4)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    dev, bs = "cuda", 16
    n_q, n_kv, hd = a.heads, a.kv_heads, a.head_dim
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tq = F.prefill_tile_tokens(n_q, n_kv)
    for n in (int(x) for x in a.lens.split(",")):
        S, T = a.seqs, a.seqs * n
        maxb = (n + bs - 1) // bs
        nb = S * maxb
        q = torch.randn(T, n_q * hd, device=dev).to(torch.bfloat16)
        kc = torch.randn(nb, bs, n_kv, hd, device=dev).to(torch.bfloat16)
        vc = torch.randn(nb, bs, n_kv, hd, device=dev).to(torch.bfloat16)
        bt = torch.randperm(nb, device=dev).view(S, maxb).int()
        rows = [s for s in range(S) for _ in range(n)]
        pos = [p for _ in range(S) for p in range(n)]
        bt_row = torch.tensor(rows, dtype=torch.int32, device=dev)
        ctx = torch.tensor([p + 1 for p in pos], dtype=torch.int32, device=dev)
        tiles, covered = F.build_prefill_tiles(rows, pos, tq)
        tiles_d = tiles.to(dev)
        out_a = torch.empty(T, n_q * hd, dtype=torch.bfloat16, device=dev)
        out_b = torch.empty_like(out_a)
        t_tok = timed(lambda: F.paged_attention(q, kc, vc, bt, bt_row, ctx, n_q, n_kv, hd, out=out_a), flush, a.iters)
        t_tile = timed(lambda: F.prefill_attention(q, kc, vc, bt, tiles_d, len(tiles), n_q, n_kv, hd, out_b), flush, a.iters)
        torch.cuda.synchronize()
        err = float((out_a.float() - out_b.float()).abs().max())
        row_bytes = 2 * n_kv * hd * 2                                   # K and V of one cached token, all kv heads
        b_tok = S * sum(p + 1 for p in range(n)) * row_bytes
        b_tile = S * sum(min(n, t0 + tq) for t0 in range(0, n, tq)) * row_bytes
        flops = 4.0 * S * n_q * hd * sum(p + 1 for p in range(n))
        print(f"{S} prompts x {n} tokens: per-token kernel {t_tok:.1f} us ({b_tok / 1e6:.0f} MB of K/V, "
              f"{b_tok / t_tok / 1e3:.0f} GB/s); tiled causal kernel {t_tile:.1f} us ({b_tile / 1e6:.0f} MB, "
              f"{flops / t_tile / 1e6:.0f} TFLOP/s causal); speed-up {t_tok / t_tile:.2f}x; max |diff| {err:.4f}", flush=True)


if __name__ == "__main__":
    main()
