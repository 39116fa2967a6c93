"""Expert grouped GEMMs of one Mixtral layer (8 experts, hidden 4096, ffn 14336, bf16) over tokens per expert:
GEMM-1 + SwiGLU and GEMM-2 of this package against ``torch._grouped_mm``.

    python benchmark/ops/grouped_gemm.py [--tokens 8,32,64,128,512] [--iters 20]

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
    a = ap.parse_args(argv)
    dev = "cuda"
    w13 = (torch.randn(E, 2 * I, H, device=dev) * 0.02).to(torch.bfloat16)        # runtime layout: K contiguous
    w2 = (torch.randn(E, H, I, device=dev) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for t in (int(x) for x in a.tokens.split(",")):
        T = t * E
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        offs = torch.arange(0, T + 1, t, dtype=torch.int32, device=dev)
        act = gemm.grouped_swiglu(x, w13, offs)
        t1 = timed(lambda: gemm.grouped_swiglu(x, w13, offs), flush, a.iters)
        t2 = timed(lambda: gemm.grouped_linear(act, w2, offs), flush, a.iters)
        lib_offs = offs[1:].contiguous()
        t_lib = timed(lambda: torch._grouped_mm(x, w13.transpose(1, 2), offs=lib_offs), flush, a.iters)
        gb1, gb2 = w13.numel() * 2 / 1e9, w2.numel() * 2 / 1e9
        f1, f2 = 2.0 * T * 2 * I * H, 2.0 * T * H * I
        print(f"{t} tokens/expert: GEMM-1+SwiGLU {t1:.1f} us ({gb1 / t1 * 1e6:.0f} GB/s, {f1 / t1 / 1e6:.0f} TFLOP/s); "
              f"GEMM-2 {t2:.1f} us ({gb2 / t2 * 1e6:.0f} GB/s, {f2 / t2 / 1e6:.0f} TFLOP/s); "
              f"torch._grouped_mm GEMM-1 {t_lib:.1f} us", flush=True)
    assert gemm.check_status() == 0


if __name__ == "__main__":
    main()
