"""Two ranks, two GPUs: the consumer's kernel is launched FIRST and really blocks on a flag in its own memory; the
producer's kernel, launched about 0.3 s later on the other GPU, stores rows into the consumer's buffer (peer stores over
NVLink) and then releases the flag. The consumer checks that it did block and that it sees the producer's rows complete
(a missing system-scope fence or release / acquire pair would show as stale rows). Prints one JSON line per rank."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from disagmoe_b200.ops import functional as F
from disagmoe_b200.ops import gemm
from disagmoe_b200.parallel.peer import ArenaLayout, PeerArena


def main():
    rank, lr = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    T, H, rounds = 512, 4096, 3
    L = ArenaLayout()
    L.add("rows", T * H * 2)
    L.add("flag", 4 * 4)
    arena = PeerArena.create(L.size, device=dev)
    rows = arena.view(L.offset("rows"), (T, H), torch.bfloat16)
    flag = arena.view(L.offset("flag"), (4,), torch.int32)
    z = lambda: torch.zeros(1, dtype=torch.int32, device=dev)
    status = gemm.scratch(dev).status
    w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    out = {"rank": rank, "ok": True, "blocked_s": []}
    if rank == 0:
        # producer: RMSNorm of its rows goes straight into rank 1's buffer, then rank 1's flag slot 2 is released
        dst = arena.ptr_table([1], L.offset("rows"))
        sig = arena.ptr_table([1], L.offset("flag"))
        epoch, ticket = z(), z()
        for r in range(rounds):
            x = torch.full((T, H), float(r + 1), dtype=torch.bfloat16, device=dev)
            torch.cuda.synchronize()
            dist.barrier()
            time.sleep(0.3)
            F.norm_gather(x, None, w * (r + 1), 1e-6, None, dst, 1, 0, H, T, H, signal_ptrs=sig, n_signal=1,
                          signal_slot=2, signal_epoch=epoch, ticket=ticket, status=status)
            torch.cuda.synchronize()
            dist.barrier()
    else:
        wait_epoch = z()
        copy = torch.empty_like(rows)
        for r in range(rounds):
            torch.cuda.synchronize()
            dist.barrier()
            t0 = time.time()
            # consumer first: the wait kernel spins (bounded) until the producer's release arrives, then the copy runs
            F.wait_flags(flag[2:], 1, wait_epoch, status)
            copy.copy_(rows)
            torch.cuda.synchronize()
            out["blocked_s"].append(round(time.time() - t0, 3))
            want = float(r + 1)       # rmsnorm of a constant row is 1 everywhere, times the weight r + 1
            if not bool((copy.float() == want).all()):
                out["ok"] = False
                out["bad_rows"] = int((copy.float() != want).any(1).sum())
            dist.barrier()
        out["status"] = gemm.check_status(dev)
        out["ok"] = out["ok"] and out["status"] == 0 and min(out["blocked_s"]) > 0.2
    print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
