"""Point-to-point latency of the transports between two GPUs of one node for a 512 x 4096 bf16 tensor (4 MB)
(reference: benchmark/local_comm_latency.py:12,350-357):

  torch     torch.distributed NCCL send / recv
  channel   the native NcclChannel (2-rank communicator, private stream) + its control message
  peer      a kernel of this package storing the rows straight into the peer's arena (what the fused dispatch does)

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port P \
        benchmark/local_comm_latency.py
"""
import ctypes
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from disagmoe_b200 import disagmoe_c as C
from disagmoe_b200.ops import _lib
from disagmoe_b200.parallel.peer import PeerArena


def timed(fn, iters=20):
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(float(t))
    ts.sort()
    return ts[len(ts) // 2] * 1e3


def main():
    rank, lr = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    n, H = 512, 4096
    x = torch.randn(n, H, device="cuda").to(torch.bfloat16)
    res = {}

    def torch_p2p():
        dist.send(x, 1) if rank == 0 else dist.recv(x, 0)
    for _ in range(3):
        torch_p2p()
    res["torch_nccl_us"] = timed(torch_p2p)

    uid = [C.get_nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, 0)
    ch = C.create_channel(rank, 1 - rank, uid[0])
    ch.instantiate()
    meta = C.Metadata([n, H])

    def channel_p2p():
        if rank == 0:
            ch.send(x, meta); ch.sync()
        else:
            ch.recv(meta)
    for _ in range(3):
        channel_p2p()
    res["native_channel_us"] = timed(channel_p2p)

    arena = PeerArena.create(n * H * 2 + 4096, device=torch.device("cuda", lr))
    mp = torch.arange(n, dtype=torch.int32, device="cuda")

    def peer_store():
        if rank == 0:
            _lib.check(_lib.lib().dmoe_permute_rows(
                ctypes.c_void_p(x.data_ptr()), ctypes.c_longlong(H), ctypes.c_void_p(arena.ptr(1, 0)), ctypes.c_longlong(H),
                ctypes.c_void_p(mp.data_ptr()), ctypes.c_int(n), ctypes.c_int(H), ctypes.c_int(1), ctypes.c_int(0),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "permute_rows")
    for _ in range(3):
        peer_store()
    res["peer_store_kernel_us"] = timed(peer_store)
    if rank == 0:
        mb = n * H * 2 / 1e6
        print({k: round(v, 1) for k, v in res.items()}, {k.replace("_us", "_GBs"): round(mb / v * 1e3, 1) for k, v in res.items()})
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
