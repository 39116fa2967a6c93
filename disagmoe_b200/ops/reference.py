"""Plain PyTorch restatements of every device op (any device, any float dtype; math in fp32).

They are the numerical reference of the CUDA kernels' tests, the building blocks of the fp32 CPU oracle model
and the CPU path of the ops in :mod:`disagmoe_b200.ops.functional`.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * w.float()).to(x.dtype)


def add_rmsnorm(resid: Optional[torch.Tensor], adds: List[torch.Tensor], w: torch.Tensor, eps: float
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """new_resid = resid + sum(adds) (rounded to the storage dtype); y = rmsnorm(new_resid) * w."""
    acc = None if resid is None else resid.float()
    for a in adds:
        acc = a.float() if acc is None else acc + a.float()
    dtype = resid.dtype if resid is not None else adds[0].dtype
    new = acc.to(dtype)
    return new, rmsnorm(new, w, eps)


def rope_neox(x: torch.Tensor, positions: torch.Tensor, n_heads: int, hd: int, theta: float) -> torch.Tensor:
    """x [T, n_heads*hd]; rotates pairs (d, d + hd/2) by positions * theta^(-2d/hd)."""
    T = x.shape[0]
    xf = x.float().view(T, n_heads, hd)
    half = hd // 2
    inv_freq = theta ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2.0 / hd)
    ang = positions.float()[:, None] * inv_freq[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = xf[..., :half], xf[..., half:]
    out = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    return out.reshape(T, n_heads * hd).to(x.dtype)


def rope_kv_append(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor], kcache: torch.Tensor,
                   vcache: torch.Tensor, n_q: int, n_kv: int, hd: int, theta: float) -> None:
    """In place: RoPE on q and k heads of qkv rows [q | k | v]; append k, v at flat slot ids of the paged cache
    (cache shape [num_blocks, block_size, n_kv, hd])."""
    qd, kd = n_q * hd, n_kv * hd
    qkv[:, :qd] = rope_neox(qkv[:, :qd], positions, n_q, hd, theta)
    qkv[:, qd:qd + kd] = rope_neox(qkv[:, qd:qd + kd], positions, n_kv, hd, theta)
    if slots is not None:
        ok = slots >= 0
        kflat = kcache.view(-1, n_kv * hd)
        vflat = vcache.view(-1, n_kv * hd)
        kflat[slots[ok]] = qkv[ok, qd:qd + kd].to(kcache.dtype)
        vflat[slots[ok]] = qkv[ok, qd + kd:qd + 2 * kd].to(vcache.dtype)


def paged_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                    bt_row: Optional[torch.Tensor], ctx_len: torch.Tensor, n_q: int, n_kv: int, hd: int,
                    scale: Optional[float] = None) -> torch.Tensor:
    """Token t attends to the first ctx_len[t] cached tokens of block-table row bt_row[t] (default t)."""
    T = q.shape[0]
    block_size = kcache.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    out = torch.zeros(T, n_q * hd, dtype=torch.float32, device=q.device)
    gq = n_q // n_kv
    for t in range(T):
        L = int(ctx_len[t])
        if L == 0:
            continue
        row = int(bt_row[t]) if bt_row is not None else t
        nb = (L + block_size - 1) // block_size
        blocks = block_tables[row, :nb].long()
        k = kcache[blocks].reshape(nb * block_size, n_kv, hd)[:L].float()
        v = vcache[blocks].reshape(nb * block_size, n_kv, hd)[:L].float()
        qt = q[t].float().view(n_kv, gq, hd)
        s = torch.einsum("kgd,lkd->kgl", qt, k) * scale
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("kgl,lkd->kgd", p, v)
        out[t] = o.reshape(-1)
    return out.to(q.dtype)


def route(x: torch.Tensor, norm_w: Optional[torch.Tensor], eps: float, gate_w: torch.Tensor, top_k: int,
          renormalize: bool, logit_bias: Optional[torch.Tensor] = None
          ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(y, topk_ids int32 [T,k], topk_w fp32 [T,k], logits fp32): y = rmsnorm(x) (or x), softmax -> top-k."""
    y = rmsnorm(x, norm_w, eps) if norm_w is not None else x
    logits = y.float() @ gate_w.float().T
    if logit_bias is not None:
        logits = logits + logit_bias.float().to(logits.device)
    probs = torch.softmax(logits, dim=-1)
    w, ids = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return y, ids.int(), w.float(), logits


def expert_offsets(topk_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    counts = torch.bincount(topk_ids.reshape(-1).long(), minlength=num_experts)
    offs = torch.zeros(num_experts + 1, dtype=torch.int32, device=topk_ids.device)
    offs[1:] = counts.cumsum(0).int()
    return offs


def sort_by_expert(topk_ids: torch.Tensor) -> torch.Tensor:
    """Stable counting sort of the flattened (token-major) [T*k] expert ids; returns dst position of every pair."""
    flat = topk_ids.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    pos = torch.empty_like(order)
    pos[order] = torch.arange(flat.numel(), device=flat.device)
    return pos.int()


def swiglu(h: torch.Tensor) -> torch.Tensor:
    I = h.shape[-1] // 2
    return torch.nn.functional.silu(h[..., :I].float()) * h[..., I:].float()


def moe_experts(y: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor
                ) -> torch.Tensor:
    """Weighted sum over the top-k experts; w13 [E, 2I, H] (gate rows then up rows), w2 [E, H, I]. fp32 result."""
    T, H = y.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=y.device)
    E = w13.shape[0]
    yf = y.float()
    for e in range(E):
        tok, slot = (topk_ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = swiglu(yf[tok] @ w13[e].float().T).to(y.dtype).float()
        o = (h @ w2[e].float().T).to(y.dtype).float()
        out.index_add_(0, tok, o * topk_w[tok, slot][:, None].float())
    return out


def permute_rows(src: torch.Tensor, mapping: torch.Tensor, repeat: int = 1, gather: bool = False,
                 n_out: Optional[int] = None) -> torch.Tensor:
    n = mapping.numel()
    m = mapping.long()
    if gather:
        out = torch.zeros(n, src.shape[1], dtype=src.dtype, device=src.device)
        ok = m >= 0
        out[ok] = src[m[ok]]
        return out
    out = torch.zeros(n_out if n_out is not None else n, src.shape[1], dtype=src.dtype, device=src.device)
    idx = torch.arange(n, device=src.device) // repeat
    ok = m >= 0
    out[m[ok]] = src[idx[ok]]
    return out
