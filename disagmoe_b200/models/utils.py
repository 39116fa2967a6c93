"""Metadata helpers for tests and the TP broadcast path (reference: disagmoe/models/utils.py:14-215)."""
from __future__ import annotations

import pickle
from typing import List

import torch
import torch.distributed as dist

from .attention import AttnMeta


def make_seqlens(lens: List[int]) -> List[int]:
    out = [0]
    for l in lens:
        out.append(out[-1] + l)
    return out


def make_naive_mapping(block_size: int, lens: List[int], mode: str = "block"):
    """Sequential block tables (sequence i owns consecutive blocks) or the flat slot of every token."""
    tables, slots, nxt = [], [], 0
    for l in lens:
        nb = (l + block_size - 1) // block_size
        blocks = list(range(nxt, nxt + nb))
        nxt += nb
        tables.append(blocks)
        slots.extend(blocks[p // block_size] * block_size + p % block_size for p in range(l))
    return tables if mode == "block" else slots


def make_prefill_meta(prompt_lens: List[int], block_size: int, device="cpu") -> AttnMeta:
    """Attention metadata of a pure-prefill batch with sequentially allocated blocks."""
    tables = make_naive_mapping(block_size, prompt_lens, "block")
    width = max(len(t) for t in tables)
    bt = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    pos, rows = [], []
    for i, l in enumerate(prompt_lens):
        pos.extend(range(l))
        rows.extend([i] * l)
    slots = make_naive_mapping(block_size, prompt_lens, "slot")
    t = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt, device=device)
    return AttnMeta(t(pos), t(slots, torch.int64), bt.to(device), t(rows), t([p + 1 for p in pos]),
                    num_prefill_tokens=len(pos), max_ctx=max(prompt_lens))


def pack_attn_meta(meta: AttnMeta) -> torch.Tensor:
    """Flattens the metadata into one int64 buffer (for a single broadcast to TP workers)."""
    T, (R, Wd) = meta.positions.numel(), meta.block_tables.shape
    head = torch.tensor([T, R, Wd, meta.num_prefill_tokens, meta.num_decode_tokens, meta.max_ctx], dtype=torch.int64)
    bt_row = meta.bt_row if meta.bt_row is not None else torch.arange(T)
    parts = [head, meta.positions.cpu().long(), meta.slots.cpu().long(), bt_row.cpu().long(), meta.ctx_len.cpu().long(),
             meta.block_tables.cpu().long().reshape(-1)]
    return torch.cat(parts)


def unpack_attn_meta(buf: torch.Tensor, device="cpu") -> AttnMeta:
    T, R, Wd, npf, ndc, mx = buf[:6].tolist()
    o = 6
    take = lambda n: buf[o:o + n]
    pos = buf[o:o + T]; o += T
    slots = buf[o:o + T]; o += T
    rows = buf[o:o + T]; o += T
    ctx = buf[o:o + T]; o += T
    bt = buf[o:o + R * Wd].view(R, Wd)
    return AttnMeta(pos.int().to(device), slots.long().to(device), bt.int().to(device), rows.int().to(device),
                    ctx.int().to(device), npf, ndc, mx)


def broadcast_pyobj(obj, src: int = 0, group=None, device="cpu"):
    """Broadcasts a picklable object inside a process group (size first, then the bytes)."""
    rank = dist.get_rank(group)
    if rank == src:
        data = torch.frombuffer(bytearray(pickle.dumps(obj)), dtype=torch.uint8).to(device)
        size = torch.tensor([data.numel()], dtype=torch.int64, device=device)
    else:
        size = torch.zeros(1, dtype=torch.int64, device=device)
    dist.broadcast(size, src, group=group)
    if rank != src:
        data = torch.empty(int(size), dtype=torch.uint8, device=device)
    dist.broadcast(data, src, group=group)
    return obj if rank == src else pickle.loads(data.cpu().numpy().tobytes())
