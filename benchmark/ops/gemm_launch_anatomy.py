"""Where the time of one GEMM launch goes: CTA 0 of the kernel stamps %globaltimer at its milestones when
``ops.gemm.TRACE`` points at an int64 [16] CUDA tensor (prologue, first TMA, first stage landed, last MMA, epilogue
chunk 0 step by step, end of the epilogue). Prints the mean of 10 launches per shape, microseconds after kernel entry.

    python benchmark/ops/gemm_launch_anatomy.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from disagmoe_b200.ops import gemm

DEV = "cuda"
# stamp i + 1 of the trace buffer (stamp 0 is the kernel's entry)
NAMES = ["set-up done", "first TMA issued", "first stage landed", "last MMA committed", "epilogue sees accumulator",
         "epilogue done", "tear-down reached (thread 0)", "chunk 0: TMEM read", "chunk 0: staged", "chunk 0: barrier",
         "chunk 0: rows stored", "chunk 0: second barrier", "producer: walker initialised", "producer: L2 policies",
         "producer: first stage free"]


def run(tag, fn, launches=10):
    trace = torch.zeros(16, dtype=torch.int64, device=DEV)
    gemm.TRACE = trace
    try:
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        acc = torch.zeros(len(NAMES))
        for _ in range(launches):
            trace.zero_()
            fn()
            torch.cuda.synchronize()
            t = trace.cpu()
            acc += torch.tensor([(t[i + 1] - t[0]).item() / 1e3 for i in range(len(NAMES))])
    finally:
        gemm.TRACE = None
    print(tag + ": " + ", ".join(f"{name} +{v:.2f}" for name, v in zip(NAMES, (acc / launches).tolist()))
          + " us after entry", flush=True)


def main():
    for T, F, K, bn in ((256, 6144, 64, 128), (256, 6144, 4096, 128), (32, 6144, 64, 32), (1024, 4096, 1024, 256)):
        w = torch.randn(F, K, device=DEV, dtype=torch.bfloat16) * 0.02
        x = torch.randn(T, K, device=DEV, dtype=torch.bfloat16)
        out = torch.empty(T, F, device=DEV, dtype=torch.bfloat16)
        run(f"linear T={T} F={F} K={K} tile={bn}", lambda: gemm.linear(x, w, out=out, bn=bn, splitk=1))
    G, H, I = 2, 4096, 14336
    w13 = gemm.block_weight((torch.randn(G, 2 * I, H, device=DEV) * 0.02).to(torch.bfloat16))
    x = torch.randn(512, H, device=DEV).to(torch.bfloat16)
    offs = torch.tensor([0, 250, 512], dtype=torch.int32, device=DEV)
    run("grouped SwiGLU, 2 experts x ~256 tokens", lambda: gemm.grouped_swiglu(x, w13, offs, w_blocked=True))
    assert gemm.check_status() == 0


if __name__ == "__main__":
    main()
