"""ctypes loader of ``lib/libdmoe_kernels.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`disagmoe_b200.build`. An op called with CUDA tensors raises if the library
is missing: there is no silent eager fallback on a GPU box.
"""
from __future__ import annotations

import ctypes
import os

import torch

_LIB = None
_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libdmoe_kernels.so")


class KernelError(RuntimeError):
    pass


class DmoeGemm(ctypes.Structure):
    _fields_ = [
        ("W", ctypes.c_void_p), ("X", ctypes.c_void_p), ("Y", ctypes.c_void_p), ("R", ctypes.c_void_p),
        ("offs", ctypes.c_void_p), ("recs", ctypes.c_void_p), ("bases", ctypes.c_void_p), ("ws", ctypes.c_void_p),
        ("counters", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("seg_cnt", ctypes.c_void_p), ("wait_flags", ctypes.c_void_p), ("wait_epoch", ctypes.c_void_p),
        ("signal_ptrs", ctypes.c_void_p), ("signal_epoch", ctypes.c_void_p), ("done_ticket", ctypes.c_void_p),
        ("ldx", ctypes.c_longlong), ("ldy", ctypes.c_longlong), ("ldr", ctypes.c_longlong),
        ("ws_bytes", ctypes.c_longlong),
        ("S", ctypes.c_int), ("seg_cap", ctypes.c_int), ("n_wait", ctypes.c_int), ("n_signal", ctypes.c_int),
        ("signal_slot", ctypes.c_int), ("group_regions", ctypes.c_int), ("clear_n", ctypes.c_int),
        ("clear_ptr", ctypes.c_void_p), ("fanout", ctypes.c_int),
        ("G", ctypes.c_int), ("T", ctypes.c_int), ("F", ctypes.c_int), ("K", ctypes.c_int),
        ("epi", ctypes.c_int), ("bn", ctypes.c_int), ("splitk", ctypes.c_int), ("y_f32", ctypes.c_int),
        ("shard_rows", ctypes.c_int), ("rs_bases", ctypes.c_void_p),
        ("rs_rows", ctypes.c_int), ("rs_slot", ctypes.c_int), ("rs_cap", ctypes.c_int),
        ("rope_table", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("slots", ctypes.c_void_p),
        ("kcache", ctypes.c_void_p), ("vcache", ctypes.c_void_p),
        ("n_q", ctypes.c_int), ("n_kv", ctypes.c_int), ("hd", ctypes.c_int), ("rope_max_pos", ctypes.c_int),
        ("streamk", ctypes.c_int), ("n_counters", ctypes.c_int), ("pair", ctypes.c_int),
        ("combine_vec", ctypes.c_int), ("w_blocked", ctypes.c_int),
        ("trace", ctypes.c_void_p),
    ]


_vp, _ll, _i, _f = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float


class DmoeNormGather(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("resid_in", "add", "w", "resid_out", "dst_ptrs", "wait_flags", "wait_epoch",
                                   "signal_ptrs", "signal_epoch", "ticket", "status")] + \
               [(n, _ll) for n in ("ld_in", "add_row_stride", "add_part_stride", "ld_out", "dst_row0", "ld_dst")] + \
               [("eps", _f)] + \
               [(n, _i) for n in ("n_add", "n_dst", "T", "H", "n_wait", "n_signal", "signal_slot")]


class DmoeRouteDispatch(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ("resid", "add", "norm_w", "gate_w", "logit_bias", "y", "topk_ids", "topk_w",
                                   "x_bases", "rec_bases", "cnt_bases", "flag_bases", "disp_epoch", "wait_flags",
                                   "wait_epoch", "ticket", "status")] + \
               [(n, _ll) for n in ("ld_resid", "add_slot_stride", "ld_add", "ld_y", "ld_dst")] + \
               [("eps", _f)] + \
               [(n, _i) for n in ("n_add", "T", "H", "E", "K", "renorm", "experts_per_rank", "n_dst", "my_rank",
                                  "region_cap", "n_wait", "ret_rank", "ret_rank_set")]


def lib_path() -> str:
    return _LIB_PATH


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def lib():
    """The loaded kernel library. Raises KernelError if it has not been built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(_LIB_PATH):
            raise KernelError(
                f"{_LIB_PATH} is missing: run `python -m disagmoe_b200.build` (nvcc, sm_100a) before using CUDA ops")
        _LIB = ctypes.CDLL(_LIB_PATH)
        _LIB.dmoe_gemm.argtypes = [ctypes.POINTER(DmoeGemm), ctypes.c_void_p]
        _LIB.dmoe_gemm.restype = ctypes.c_int
        _LIB.dmoe_gemm_workspace_bytes.restype = ctypes.c_longlong
        _LIB.dmoe_norm_gather.argtypes = [ctypes.POINTER(DmoeNormGather), ctypes.c_void_p]
        _LIB.dmoe_route_dispatch.argtypes = [ctypes.POINTER(DmoeRouteDispatch), ctypes.c_void_p]
        _LIB.dmoe_set_flag_wait_cycles.argtypes = [ctypes.c_longlong]
        _LIB.dmoe_set_flag_wait_cycles.restype = None
    return _LIB


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = 0   # entry-point calls that launched kernels of this library (a graph replay adds its captured count)


TIMELINE = None   # a list while a timeline is being taken: (label, CUDA event recorded right after the launch)
TAG = ""          # set by callers to tell launches of one entry point apart (QKV / o_proj / LM head GEMM ...)


def start_timeline() -> None:
    """From now on every launch made through :func:`check` is followed by a timing event on the current stream (eager
    launches only: do not capture a graph while a timeline is on)."""
    global TIMELINE
    TIMELINE = []
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    TIMELINE.append(("start", ev))


def stop_timeline():
    """Ends the timeline and returns {label: (launches, total ms)}: the device time between the end of the previous
    launch and the end of this one, i.e. the kernel's run time including any wait on peers' flags inside it."""
    global TIMELINE
    tl, TIMELINE = TIMELINE, None
    torch.cuda.synchronize()
    out = {}
    for (_, a), (name, b) in zip(tl[:-1], tl[1:]):
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + a.elapsed_time(b))
    return out


def check(code: int, what: str):
    global LAUNCHES
    if code != 0:
        raise KernelError(f"{what} failed with code {code}")
    LAUNCHES += 1
    if TIMELINE is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        TIMELINE.append(((TAG + ":" if TAG else "") + what, ev))


def add_launches(n: int):
    global LAUNCHES
    LAUNCHES += n


def ptr(t):
    return 0 if t is None else t.data_ptr()
