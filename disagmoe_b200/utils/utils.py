"""Small helpers shared by the engine, the controller and the benchmarks
(reference: disagmoe/utils/utils.py:19-192)."""
from __future__ import annotations

import os
import socket
import time
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple, Union

import torch
from torch import Tensor

from .logger import get_logger


def _recorder_fns():
    try:
        from .. import disagmoe_c
        return disagmoe_c.range_push, disagmoe_c.range_pop
    except Exception:
        return (lambda msg: None), (lambda: None)


def get_nccl_unique_id():
    """A fresh NCCL unique id as bytes (needs a CUDA build of torch; raises on CPU-only hosts)."""
    from torch.cuda.nccl import unique_id
    return unique_id()


def get_nccl_url_from_uid(uid) -> str:
    h = 0
    for b in bytes(uid):
        h = (h * 256 + b) % 10007
    return f"{os.environ.get('MASTER_ADDR', '127.0.0.1')}:{int(os.environ.get('MASTER_PORT', '26500')) + h}"


class Counter:
    """Wrapping integer iterator."""

    def __init__(self, start: int = 0, end: int = 2_000_000_000, step: int = 1):
        self.start, self.counter, self.end, self.step = start, start, end, step

    def __iter__(self):
        return self

    def __next__(self) -> int:
        i = self.counter
        self.counter += self.step
        if self.counter >= self.end:
            self.counter = 0
        return i

    def reset(self) -> None:
        self.counter = self.start


def get_ip() -> str:
    ip = os.environ.get("HOST_IP")
    if ip:
        return ip
    for fam, probe in ((socket.AF_INET, ("10.255.255.255", 1)), (socket.AF_INET6, ("fd00::1", 1))):
        s = None
        try:
            s = socket.socket(fam, socket.SOCK_DGRAM)
            s.connect(probe)   # no packet is sent for a datagram socket
            return s.getsockname()[0]
        except Exception:
            pass
        finally:
            if s is not None:
                s.close()
    return "127.0.0.1"


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@contextmanager
def nvtx_range_cuda(msg, *args, **kwargs):
    torch.cuda.nvtx.range_push(msg.format(*args, **kwargs))
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


@contextmanager
def nvtx_range(msg, *args, **kwargs):
    """A range in the native recorder (a no-op unless ENABLE_NVTX=1)."""
    push, pop = _recorder_fns()
    push(msg.format(*args, **kwargs))
    try:
        yield
    finally:
        pop()


class CudaRangeEvent:
    def __init__(self, enable_timing: bool = False):
        self._start = torch.cuda.Event(enable_timing=enable_timing)
        self._end = torch.cuda.Event(enable_timing=enable_timing)

    def start(self):
        self._start.record()

    def end(self):
        self._end.record()

    def timing(self) -> float:
        return self._start.elapsed_time(self._end)


def make_seqlens_list(lens: Union[List[int], Tensor], dst: Optional[List[int]] = None) -> Optional[List[int]]:
    """Exclusive prefix sums [0, l0, l0+l1, ...]; None for an empty input."""
    if isinstance(lens, Tensor):
        lens = lens.view(-1).tolist()
    if len(lens) == 0:
        return None
    if dst is None:
        dst = [0] * (len(lens) + 1)
    assert len(dst) == len(lens) + 1
    run = 0
    dst[0] = 0
    for i, l in enumerate(lens):
        run += int(l)
        dst[i + 1] = run
    return dst


def make_seqlens_cuda_tensor(lens: Union[List[int], Tensor], device="cuda") -> Optional[Tensor]:
    out = make_seqlens_list(lens)
    return None if out is None else torch.tensor(out, dtype=torch.int32, device=device)


def get_graph_batch_size(batch_size: int, graph_batch_sizes: List[int]) -> Tuple[int, int]:
    """Index and size of the smallest captured bucket that fits ``batch_size``."""
    for i, size in enumerate(graph_batch_sizes):
        if size >= batch_size:
            return i, size
    raise ValueError(f"no captured graph fits batch size {batch_size} (largest {graph_batch_sizes[-1]})")


def graph_batch_sizes(max_bs: int, stride: int, ep_size: int = 1) -> List[int]:
    """Bucket rule of the CUDA-graph executor: 1, then multiples of the stride up to max_bs
    (reference: disagmoe/executor/executor.py:145-148)."""
    first = max(stride, ep_size)
    sizes = [1] + list(range(first, max_bs + 1, stride))
    if sizes[-1] != max_bs:
        sizes.append(max_bs)
    return sizes


@dataclass
class StepInfo:
    start_timestamp_ms: float
    end_timestamp_ms: float
    batch_size: int
    layer_id: int
    internal_layer_id: int
    pool_snapshot: Dict[int, int] = field(default_factory=dict)
    thread_id: int = -1
    process_id: int = -1


def time_ms() -> float:
    return time.time() * 1000


class Timer:
    """Named wall-clock timers in milliseconds."""

    def __init__(self):
        self.timers: Dict[str, float] = {}
        self._open: Dict[str, int] = {}

    def start(self, name: str) -> None:
        self._open[name] = time.perf_counter_ns()

    def stop(self, name: str) -> float:
        t0 = self._open.pop(name)
        self.timers[name] = (time.perf_counter_ns() - t0) / 1e6
        return self.timers[name]

    def get(self, name: str) -> Optional[float]:
        return self.timers.get(name)
