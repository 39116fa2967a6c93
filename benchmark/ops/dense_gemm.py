"""Decode-size dense GEMMs (QKV and o_proj + residual of the Mixtral shape) against cuBLAS, with a tile / split-K sweep.

    python benchmark/ops/dense_gemm.py [--tokens 64,128,256,512] [--sweep]

Every measurement is one CUDA graph of 24 launches over 24 distinct weight matrices (so weights always come from HBM,
as in a decoder stack, and host launch overhead is excluded), timed with CUDA events around graph replays, best of 4.
cuBLAS goes through ``torch.matmul`` / ``torch.addmm`` in the same harness. ``--sweep`` also tries every token tile
(32..256) and split-K factor (1..8) and prints the four fastest.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from disagmoe_b200.ops import gemm

N_WEIGHTS = 24


def bench(fn, n=N_WEIGHTS, reps=4):
    for i in range(n):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i)
    for _ in range(12):      # clocks and caches settle before anything is timed
        g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / n * 1e3)
    return best


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="64,128,256,512")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--tp", type=int, default=1, help="shapes of one rank of a tensor-parallel attention group: QKV has "
                    "6144 / tp output features, o_proj 4096 / tp input features and no residual (reduce-scatter epilogue)")
    ap.add_argument("--hbm-gbs", type=float, default=6549.0, help="copy bandwidth for the weight-streaming floor")
    a = ap.parse_args(argv)
    dev = "cuda"
    shapes = (("qkv", 6144, 4096, False), ("o_proj+residual", 4096, 4096, True)) if a.tp == 1 else \
        ((f"qkv/tp{a.tp}", 6144 // a.tp, 4096, False), (f"o_proj/tp{a.tp}", 4096, 4096 // a.tp, False))
    for name, F, K, resid in shapes:
        ws = [torch.randn(F, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(N_WEIGHTS)]
        for T in (int(t) for t in a.tokens.split(",")):
            x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
            r = torch.randn(T, F, device=dev, dtype=torch.bfloat16) if resid else None
            out = torch.empty(T, F, device=dev, dtype=torch.bfloat16)

            def lib(i):
                if resid:
                    torch.addmm(r, x, ws[i].T, out=out)
                else:
                    torch.matmul(x, ws[i].T, out=out)

            t_lib = bench(lib)
            t_own = bench(lambda i: gemm.linear(x, ws[i], residual=r, out=out))
            line = (f"{name} T={T}: this kernel {t_own:.1f} us, cuBLAS {t_lib:.1f} us, weight-streaming floor "
                    f"{F * K * 2 / a.hbm_gbs / 1e3:.1f} us")
            if a.sweep:
                res = []
                for bn in (32, 64, 128, 256):
                    if bn > max(32, T):
                        continue
                    for sk in (1, 2, 3, 4, 6, 8):
                        try:
                            res.append((bench(lambda i: gemm.linear(x, ws[i], residual=r, out=out, bn=bn, splitk=sk)), bn, sk))
                        except Exception:
                            pass
                res.sort()
                line += "; fastest (us, tile, split-K): " + str([(round(t, 1), bn, sk) for t, bn, sk in res[:4]])
            print(line, flush=True)
    assert gemm.check_status() == 0


if __name__ == "__main__":
    main()
