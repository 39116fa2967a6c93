"""Peer-memory arenas: one device buffer per rank, laid out identically everywhere and mapped into every peer.

Kernels address a peer's copy of a sub-buffer as ``arena.ptr(rank, offset)`` and read / write it with ordinary
loads and stores that travel over NVLink / NVSwitch. Handles are exchanged once at start-up (CUDA IPC through
PyTorch's storage sharing); the hot path never touches the host. For tests, :meth:`PeerArena.emulated` builds
several "ranks" on one GPU whose arenas simply point at each other.

This is the data plane that replaces the reference's per-edge 2-rank NCCL communicators
(csrc/muhelper/comm.cpp:39-78, ids minted at disagmoe/frontend/controller.py:143-153).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from ..ops import _lib


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class _RawCudaBuffer:
    """Exposes a raw device address through ``__cuda_array_interface__`` so that torch can view it as a tensor."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _wrap_device_memory(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """uint8 tensor over ``nbytes`` at device address ``ptr`` (memory owned by the kernel library, never freed by
    torch). The tensor is labelled with ``device``: for a mapped peer block that is the device whose kernels use it."""
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)


class ArenaLayout:
    """Names -> (offset, nbytes) with 256-byte alignment; identical on every rank."""

    def __init__(self):
        self.entries = {}
        self.size = 0

    def add(self, name: str, nbytes: int) -> int:
        off = self.size
        self.entries[name] = (off, nbytes)
        self.size = _align(off + nbytes)
        return off

    def offset(self, name: str) -> int:
        return self.entries[name][0]


class PeerArena:
    def __init__(self, rank: int, world: int, local: torch.Tensor, peers: List[torch.Tensor], keep=None):
        self.rank, self.world, self.local, self.peers = rank, world, local, peers
        self._keep = keep

    # ---- construction --------------------------------------------------------------------------------------
    @staticmethod
    def create(nbytes: int, group=None, device: Optional[torch.device] = None) -> "PeerArena":
        """Collective over ``group``: allocates the local arena, exchanges CUDA IPC handles, maps every peer.

        The arena is allocated and mapped by the kernel library itself: a peer's block has to be opened with this
        process's own device current so that kernels running on it may load from and store to the block."""
        import torch.distributed as dist
        device = device or torch.device("cuda", torch.cuda.current_device())
        assert torch.cuda.current_device() == device.index, "make the arena's device current first"
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        nbytes = _align(nbytes, 2 << 20)
        lib = _lib.lib()
        p = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.dmoe_peer_alloc(ctypes.c_longlong(nbytes), ctypes.byref(p), handle), "dmoe_peer_alloc")
        _lib.LAUNCHES -= 1
        gathered = [None] * world
        dist.all_gather_object(gathered, (handle.raw, nbytes), group=group)
        ptrs = []
        for r, (h, n) in enumerate(gathered):
            if r == rank:
                ptrs.append(p.value)
                continue
            q = ctypes.c_void_p()
            _lib.check(lib.dmoe_peer_open(ctypes.c_char_p(h), ctypes.byref(q)), "dmoe_peer_open")
            _lib.LAUNCHES -= 1
            ptrs.append(q.value)
        peers = [_wrap_device_memory(ptrs[r], nbytes, device) for r in range(world)]
        dist.barrier(group=group)
        return PeerArena(rank, world, peers[rank], peers, keep=ptrs)

    @staticmethod
    def emulated(world: int, nbytes: int, device="cuda") -> List["PeerArena"]:
        """``world`` arenas on one device that see each other (single-process emulation of a multi-GPU group)."""
        bufs = [torch.zeros(_align(nbytes), dtype=torch.uint8, device=device) for _ in range(world)]
        return [PeerArena(r, world, bufs[r], bufs) for r in range(world)]

    # ---- addressing ----------------------------------------------------------------------------------------
    def ptr(self, rank: int, offset: int = 0) -> int:
        return self.peers[rank].data_ptr() + offset

    def view(self, offset: int, shape, dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        """Typed view of a sub-buffer of this rank's arena (or, with ``rank``, of a peer's mapping)."""
        buf = self.local if rank is None else self.peers[rank]
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return buf[offset:offset + nbytes].view(dtype).view(*shape)

    def ptr_table(self, ranks: List[int], offset: int) -> torch.Tensor:
        """Device int64 tensor of the addresses of one sub-buffer on the given ranks (a kernel's pointer table)."""
        return torch.tensor([self.ptr(r, offset) for r in ranks], dtype=torch.int64, device=self.local.device)
