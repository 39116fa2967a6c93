"""Expert grouped GEMMs of one Mixtral layer (8 experts, hidden 4096, ffn 14336, bf16) over tokens per expert:
GEMM-1 + SwiGLU and GEMM-2 of this package against ``torch._grouped_mm``.

    python benchmark/ops/grouped_gemm.py [--tokens 8,32,64,128,512] [--iters 20] [--experts 8] [--ragged 0.06]

``--experts 2`` is the shape of one expert GPU of the 8-GPU layout (2 local experts); ``--ragged f`` jitters the group
sizes by +-f around the mean, as routing does. Every case runs with the stream-K work distribution and with whole
tiles per CTA, and GEMM-2 additionally at both token-tile widths.

CUDA-event timing, median of ``--iters``, a 256 MB buffer is written between iterations (L2 flush). Prints the time,
the weight-streaming rate (GB/s of expert weights) and the FLOP rate of every case.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from disagmoe_b200.ops import gemm

E, H, I = 8, 4096, 14336


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
    return ts[len(ts) // 2] * 1e3      # us


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="8,32,64,128,512", help="tokens per expert")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--experts", type=int, default=E, help="local experts (groups) of the launch")
    ap.add_argument("--ragged", type=float, default=0.0, help="relative jitter of the group sizes around the mean")
    ap.add_argument("--only", default="", help="run one variant only (for profilers): g1s / g1w / g1w256 / g1p128 / g1p256 "
                    "(GEMM-1: stream-K, whole tiles, whole 256-token tiles, CTA pairs) or g2s128 / g2s256 / g2w128 / g2w256 "
                    "/ g2p128 / g2p256 (GEMM-2); g1b / g2b: whole tiles over tile-blocked weights")
    a = ap.parse_args(argv)
    dev = "cuda"
    G = a.experts
    w13 = (torch.randn(G, 2 * I, H, device=dev) * 0.02).to(torch.bfloat16)        # runtime layout: K contiguous
    w2 = (torch.randn(G, H, I, device=dev) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    gen = torch.Generator().manual_seed(0)
    for t in (int(x) for x in a.tokens.split(",")):
        sizes = [max(1, int(round(t * (1 + a.ragged * (2 * float(torch.rand(1, generator=gen)) - 1))))) for _ in range(G)]
        T = sum(sizes)
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        offs = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device=dev)
        act = gemm.grouped_swiglu(x, w13, offs)
        if a.only:
            v = a.only
            bn = int(v[3:]) if len(v) > 3 else 0
            blocked = v[2] == "b"       # g1b / g2b: whole tiles over tile-blocked weight stacks
            if v.startswith("g1"):
                wa = gemm.block_weight(w13) if blocked else w13
                fn = lambda: gemm.grouped_swiglu(x, wa, offs, bn=bn, streamk=v[2] == "s", pair=v[2] == "p", w_blocked=blocked)
            else:
                wa = gemm.block_weight(w2) if blocked else w2
                fn = lambda: gemm.grouped_linear(act, wa, offs, bn=bn, streamk=v[2] == "s", pair=v[2] == "p", w_blocked=blocked)
            print(f"{G} experts x ~{t} tokens, {v}: {timed(fn, flush, a.iters):.1f} us", flush=True)
            continue
        res = {}
        for sk in (True, False):
            res[("g1", sk)] = timed(lambda: gemm.grouped_swiglu(x, w13, offs, streamk=sk), flush, a.iters)
            for bn in (128, 256):
                res[("g2", sk, bn)] = timed(lambda: gemm.grouped_linear(act, w2, offs, bn=bn, streamk=sk), flush, a.iters)
        # CTA pairs (cta_group::2): 256 weight rows per MMA, the token tile split between the two CTAs' shared memories
        w13b, w2b = gemm.block_weight(w13), gemm.block_weight(w2)
        res[("g1b",)] = timed(lambda: gemm.grouped_swiglu(x, w13b, offs, streamk=False, w_blocked=True), flush, a.iters)
        res[("g2b",)] = timed(lambda: gemm.grouped_linear(act, w2b, offs, streamk=False, w_blocked=True), flush, a.iters)
        del w13b, w2b
        res[("g1", False, 256)] = timed(lambda: gemm.grouped_swiglu(x, w13, offs, bn=256, streamk=False), flush, a.iters)
        for bn in (128, 256):
            res[("g1p", bn)] = timed(lambda: gemm.grouped_swiglu(x, w13, offs, bn=bn, pair=True), flush, a.iters)
            res[("g2p", bn)] = timed(lambda: gemm.grouped_linear(act, w2, offs, bn=bn, pair=True), flush, a.iters)
        lib_offs = offs[1:].contiguous()
        t_lib = timed(lambda: torch._grouped_mm(x, w13.transpose(1, 2), offs=lib_offs), flush, a.iters)
        t_lib2 = timed(lambda: torch._grouped_mm(act, w2.transpose(1, 2), offs=lib_offs), flush, a.iters)
        gb1, gb2 = w13.numel() * 2 / 1e9, w2.numel() * 2 / 1e9
        f1, f2 = 2.0 * T * 2 * I * H, 2.0 * T * H * I
        t1 = res[("g1", True)]
        t2 = min(res[("g2", True, 128)], res[("g2", True, 256)])
        print(f"{G} experts x ~{t} tokens (sizes {sizes if G <= 8 else '...'}): "
              f"GEMM-1+SwiGLU stream-K {t1:.1f} us ({gb1 / t1 * 1e6:.0f} GB/s, {f1 / t1 / 1e6:.0f} TFLOP/s), whole tiles "
              f"{res[('g1', False)]:.1f} us (256-token tiles {res[('g1', False, 256)]:.1f}); GEMM-2 stream-K bn128 {res[('g2', True, 128)]:.1f} / bn256 "
              f"{res[('g2', True, 256)]:.1f} us (best {gb2 / t2 * 1e6:.0f} GB/s, {f2 / t2 / 1e6:.0f} TFLOP/s), whole tiles "
              f"bn128 {res[('g2', False, 128)]:.1f} / bn256 {res[('g2', False, 256)]:.1f} us; CTA pairs GEMM-1 bn128 "
              f"{res[('g1p', 128)]:.1f} / bn256 {res[('g1p', 256)]:.1f} us ({f1 / min(res[('g1p', 128)], res[('g1p', 256)]) / 1e6:.0f} "
              f"TFLOP/s), GEMM-2 bn128 {res[('g2p', 128)]:.1f} / bn256 {res[('g2p', 256)]:.1f} us "
              f"({f2 / min(res[('g2p', 128)], res[('g2p', 256)]) / 1e6:.0f} TFLOP/s); torch._grouped_mm "
              f"GEMM-1 {t_lib:.1f} us, GEMM-2 {t_lib2:.1f} us; tile-blocked weights, whole tiles: GEMM-1 "
              f"{res[('g1b',)]:.1f} us, GEMM-2 {res[('g2b',)]:.1f} us", flush=True)
    assert gemm.check_status() == 0


if __name__ == "__main__":
    main()
