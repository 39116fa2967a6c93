"""Receiving side of the cross-node latency benchmark (see common.py): receives, acknowledges, repeats."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import C, RECVER_DEV, SENDER_DEV, make_tensor, meta_for, parse, setup   # noqa: E402

import torch


def main(argv=None):
    a = parse(argv)
    setup(a)
    data = C.create_socket_channel(RECVER_DEV, SENDER_DEV, False, 2)
    ack = C.create_socket_channel(RECVER_DEV, SENDER_DEV, True, 3)
    data.instantiate()
    ack.instantiate()
    t = make_tensor(a)
    empty = torch.zeros(1, 8, dtype=torch.float32)
    m, me = meta_for(t), meta_for(empty)
    ch = tg = dist = None
    if a.transport != "socket":
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", a.sender_host)
        os.environ.setdefault("MASTER_PORT", "29533")
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", rank=1, world_size=2, device_id=torch.device("cuda", 0))
        tg = torch.empty_like(t, device="cuda")
        if a.transport == "channel":
            raw = data.recv(meta_for(torch.zeros(1, 128)))
            uid = bytes(raw.view(-1).to(torch.uint8).tolist())
            ch = C.create_channel(RECVER_DEV, SENDER_DEV, uid)
            C.instantiate_channels([ch])
    n = 0
    # the sender alternates: warm-up pairs (tensor, empty), then `iters` tensors, then `iters` empties, then a stop row
    plan = ["t", "e"] * a.warmup + ["t"] * a.iters + ["e"] * a.iters
    for kind in plan:
        if kind == "t" and a.transport == "nccl":
            dist.recv(tg, 0)
            torch.cuda.synchronize()
        elif kind == "t" and a.transport == "channel":
            ch.recv(m)
            ch.sync()
        elif kind == "t":
            got = data.recv(m)
            assert got.shape == t.shape
        else:
            data.recv(me)
        ack.send(empty, me)
        n += 1
    stop = data.recv(me)
    assert float(stop[0, 0]) == -1.0
    print(f"receiver done: {n} transfers")
    return n


if __name__ == "__main__":
    main()
