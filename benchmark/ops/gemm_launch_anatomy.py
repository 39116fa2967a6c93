"""Where the time of one GEMM launch goes: CTA 0 of the kernel stamps %globaltimer at its milestones when
``ops.gemm.TRACE`` points at an int64 [16] CUDA tensor (prologue, first TMA, first stage landed, last MMA, epilogue
chunk 0 step by step, end of the epilogue). Prints the mean of 10 launches per shape, microseconds after kernel entry.

    python benchmark/ops/gemm_launch_anatomy.py
"""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch
from disagmoe_b200.ops import gemm
dev = "cuda"
names = ["setup", "first TMA issued", "first stage landed", "last MMA committed", "epilogue sees acc", "epilogue done", "teardown", "c0 tmem read", "c0 staged", "c0 barrier", "c0 stored", "c0 barrier2", "walker init", "policies", "first empty wait"]
def run(tag, fn):
    tr = torch.zeros(16, dtype=torch.int64, device=dev)
    gemm.TRACE = tr
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    acc = torch.zeros(15)
    n = 10
    for _ in range(n):
        tr.zero_(); fn(); torch.cuda.synchronize()
        t = tr.cpu()
        acc += torch.tensor([(t[i + 1] - t[0]).item() / 1e3 for i in range(15)])
    gemm.TRACE = None
    print(tag + ": " + ", ".join(f"{nm} +{v:.2f}" for nm, v in zip(names, (acc / n).tolist())) + " us after entry", flush=True)
for T, F, K, bn in ((256, 6144, 64, 128), (256, 6144, 4096, 128), (32, 6144, 64, 32), (1024, 4096, 1024, 256)):
    w = torch.randn(F, K, device=dev, dtype=torch.bfloat16) * 0.02
    x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
    out = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
    run(f"linear T={T} F={F} K={K} bn={bn}", lambda: gemm.linear(x, w, out=out, bn=bn, splitk=1))
G, H, I = 2, 4096, 14336
w13 = gemm.block_weight((torch.randn(G, 2 * I, H, device=dev) * 0.02).to(torch.bfloat16))
x = torch.randn(512, H, device=dev).to(torch.bfloat16)
offs = torch.tensor([0, 250, 512], dtype=torch.int32, device=dev)
run("grouped swiglu 2 x 256", lambda: gemm.grouped_swiglu(x, w13, offs, w_blocked=True))
