"""Sending side of the cross-node latency benchmark (see common.py). Start recver.py first.

    python benchmark/remote_comm_latency/recver.py --sender-host A --recver-host B --transport socket
    python benchmark/remote_comm_latency/sender.py --sender-host A --recver-host B --transport socket
"""
import os
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import C, RECVER_DEV, SENDER_DEV, make_tensor, meta_for, parse, setup   # noqa: E402

import torch


def main(argv=None):
    a = parse(argv)
    setup(a)
    data = C.create_socket_channel(SENDER_DEV, RECVER_DEV, True, 2)       # sender -> receiver, rows
    ack = C.create_socket_channel(SENDER_DEV, RECVER_DEV, False, 3)       # receiver -> sender, 1-element acks
    ack.instantiate()
    data.instantiate()
    t = make_tensor(a)
    empty = torch.zeros(1, 8, dtype=torch.float32)
    m, me = meta_for(t), meta_for(empty)

    def round_trip(x, mx):
        t0 = time.perf_counter()
        data.send(x, mx)
        ack.recv(me)
        return (time.perf_counter() - t0) * 1e6

    if a.transport != "socket":
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", a.sender_host)
        os.environ.setdefault("MASTER_PORT", "29533")
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", rank=0, world_size=2, device_id=torch.device("cuda", 0))
        tg = t.cuda()
        if a.transport == "channel":
            uid = C.get_nccl_unique_id()
            data.send(torch.frombuffer(bytearray(uid), dtype=torch.uint8).float().view(1, -1), meta_for(torch.zeros(1, len(uid))))
            ch = C.create_channel(SENDER_DEV, RECVER_DEV, uid)
            C.instantiate_channels([ch])

        def round_trip(x, mx):                                            # noqa: F811
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            if x is t:
                if a.transport == "nccl":
                    dist.send(tg, 1)
                else:
                    ch.send(tg, m)
                torch.cuda.synchronize()
            else:
                data.send(x, mx)
            ack.recv(me)
            return (time.perf_counter() - t0) * 1e6

    for _ in range(a.warmup):
        round_trip(t, m)
        round_trip(empty, me)
    full = [round_trip(t, m) for _ in range(a.iters)]
    base = [round_trip(empty, me) for _ in range(a.iters)]
    one_way = statistics.median(full) - statistics.median(base)
    mb = t.numel() * t.element_size() / 1e6
    print(f"{a.transport}: {mb:.1f} MB one way in {one_way:.1f} us ({mb / max(one_way, 1e-9) * 1e6 / 1e3:.2f} GB/s); "
          f"empty round trip {statistics.median(base):.1f} us")
    data.send(torch.full((1, 8), -1.0), me)                               # tells the receiver to stop
    return one_way


if __name__ == "__main__":
    main()
