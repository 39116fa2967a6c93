"""Expert MLP cost vs batch size for several model shapes (reference: benchmark/ops/expert.py:17,68-76).

Times the fused-w13 SwiGLU MLP of ONE expert (GEMM-1 + SiLU-mul fused, GEMM-2) on the tcgen05 kernel for batches
4 ... 512 and (hidden, intermediate) in {(6k,16k), (4k,12k), (5k,8k), (7k,2k)}; CUDA events, L2 flushed between
iterations; prints one line per point and writes a CSV (and a plot when matplotlib is installed)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from benchmark.plotter.common import save_series
from disagmoe_b200.ops import gemm

SHAPES = [(6144, 16384), (4096, 12288), (5120, 8192), (7168, 2048)]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="reports/expert_mlp.png")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    series = {}
    for H, I in SHAPES:
        w13 = (torch.randn(2 * I, H, device="cuda") * 0.02).to(torch.bfloat16)
        w2 = (torch.randn(H, I, device="cuda") * 0.02).to(torch.bfloat16)
        xs, ys = [], []
        for bs in (4, 8, 16, 32, 64, 128, 256, 512):
            x = torch.randn(bs, H, device="cuda").to(torch.bfloat16)
            run = lambda: gemm.linear(gemm.swiglu_linear(x, w13), w2)
            for _ in range(3):
                run()
            ts = []
            for _ in range(a.iters):
                flush.zero_()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(); run(); e.record()
                torch.cuda.synchronize()
                ts.append(s.elapsed_time(e))
            ts.sort()
            ms = ts[len(ts) // 2]
            gbs = (w13.numel() + w2.numel()) * 2 / ms / 1e6
            print(f"H={H} I={I} batch={bs}: {ms * 1e3:.1f} us  ({gbs:.0f} GB/s of weights)")
            xs.append(bs); ys.append(ms * 1e3)
        series[f"H{H}/I{I}"] = (xs, ys)
    print(save_series(a.out, series, "expert MLP time", "batch", "us"))


if __name__ == "__main__":
    main()
