"""Shared pieces of the cross-node point-to-point latency benchmark (reference: benchmark/remote_comm_latency/*).

Two processes, normally on two nodes: ``sender.py`` pushes a 512 x 4096 bf16 tensor (4 MB) to ``recver.py`` over

  socket    the runtime's TCP message channel (what carries metadata and, on CPU, the rows themselves)
  nccl      torch.distributed NCCL send / recv (GPUs)
  channel   the runtime's NcclChannel + its control message (GPUs)

The receiver acknowledges every transfer on the control socket; the sender reports the median round trip minus the
median empty round trip, i.e. the one-way transfer cost."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from disagmoe_b200 import disagmoe_c as C

SHAPE = (512, 4096)
SENDER_DEV, RECVER_DEV = 0, 1


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sender-host", default="127.0.0.1")
    ap.add_argument("--recver-host", default="127.0.0.1")
    ap.add_argument("--transport", default="socket", choices=["socket", "nccl", "channel"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=SHAPE[0])
    ap.add_argument("--hidden", type=int, default=SHAPE[1])
    ap.add_argument("--port-base", type=int, default=0)
    return ap.parse_args(argv)


def setup(a):
    C.set_inproc_transport(False)
    C.set_port_base(a.port_base)
    C.set_hosts(os.getpid(), {SENDER_DEV: a.sender_host, RECVER_DEV: a.recver_host})


def meta_for(t):
    m = C.Metadata()
    m.shape = list(t.shape)
    m.dtype = "bf16" if t.dtype == torch.bfloat16 else "fp32"
    return m


def make_tensor(a, device="cpu"):
    g = torch.Generator().manual_seed(7)
    return torch.rand(a.rows, a.hidden, generator=g).to(torch.bfloat16).to(device)
