"""Device ops of the decoder other than the GEMMs: CUDA tensors run the sm_100a kernels of
``csrc/kernels/{elementwise,attention,moe}.cu``; CPU tensors run the PyTorch restatements of
:mod:`disagmoe_b200.ops.reference` (fp32 CPU configuration, tests).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from . import _lib, reference
from .gemm import scratch

c_ll = ctypes.c_longlong
c_int = ctypes.c_int
c_float = ctypes.c_float
c_vp = ctypes.c_void_p


def _vp(t):
    return c_vp(0 if t is None else t.data_ptr())


def _st():
    return c_vp(_lib.stream_ptr())


def add_rmsnorm(resid: Optional[torch.Tensor], add: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                resid_out: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
                want_resid: bool = True) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """new_resid = resid + add.sum(1); y = rmsnorm(new_resid) * w.

    resid [T, H] or None; add None, [T, H] or [T, P, H] (P partial outputs per token, e.g. one per top-k slot).
    Returns (new_resid or None, y).
    """
    ref = resid if resid is not None else add
    T, H = ref.shape[0], ref.shape[-1]
    if add is not None and add.dim() == 2:
        add = add.unsqueeze(1)
    if not ref.is_cuda:
        adds = [] if add is None else [add[:, p] for p in range(add.shape[1])]
        new, yy = reference.add_rmsnorm(resid, adds, w, eps)
        if resid_out is not None:
            resid_out.copy_(new)
            new = resid_out
        if y is not None:
            y.copy_(yy)
            yy = y
        return (new if want_resid else None), yy
    if y is None:
        y = torch.empty(T, H, dtype=torch.bfloat16, device=ref.device)
    need_resid_out = want_resid and (add is not None)
    if need_resid_out and resid_out is None:
        resid_out = torch.empty(T, H, dtype=torch.bfloat16, device=ref.device)
    n_add = 0 if add is None else add.shape[1]
    _lib.check(_lib.lib().dmoe_add_rmsnorm(
        _vp(resid), _vp(add), c_int(n_add), c_ll(add.stride(0) if add is not None else 0),
        c_ll(add.stride(1) if add is not None else 0), _vp(w), c_float(eps), _vp(resid_out if need_resid_out else None),
        _vp(y), c_int(T), c_int(H), c_ll(resid.stride(0) if resid is not None else 0),
        c_ll(resid_out.stride(0) if need_resid_out else 0), c_ll(y.stride(0)), _st()), "dmoe_add_rmsnorm")
    if not want_resid:
        return None, y
    return (resid_out if need_resid_out else resid), y


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return add_rmsnorm(x, None, w, eps, y=out, want_resid=False)[1]


def rope_kv_append(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor], kcache: torch.Tensor,
                   vcache: torch.Tensor, n_q: int, n_kv: int, hd: int, theta: float) -> None:
    """In place neox RoPE on the q/k heads of qkv rows [q | k | v], then append k, v to the paged cache
    ([num_blocks, block_size, n_kv, hd]) at flat slots (int64, < 0 = skip)."""
    if not qkv.is_cuda:
        return reference.rope_kv_append(qkv, positions, slots, kcache, vcache, n_q, n_kv, hd, theta)
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and positions.dtype == torch.int32
    assert slots is None or slots.dtype == torch.int64
    assert kcache.is_contiguous() and vcache.is_contiguous()
    _lib.check(_lib.lib().dmoe_rope_kv_append(
        _vp(qkv), c_ll(qkv.stride(0)), _vp(positions), _vp(slots), _vp(kcache), _vp(vcache), c_int(qkv.shape[0]),
        c_int(n_q), c_int(n_kv), c_int(hd), c_float(theta), _st()), "dmoe_rope_kv_append")


def pick_attn_splits(T: int, n_kv: int, max_ctx: int, block_size: int) -> int:
    from .gemm import num_sms
    sms = num_sms()
    ctas = max(1, T * n_kv)
    if ctas >= 2 * sms or max_ctx <= 256:
        return 1
    want = (4 * sms + ctas - 1) // ctas
    return max(1, min(want, (max_ctx + 255) // 256, 64))


_attn_ws = {}


def paged_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                    bt_row: Optional[torch.Tensor], ctx_len: torch.Tensor, n_q: int, n_kv: int, hd: int,
                    out: Optional[torch.Tensor] = None, splits: int = 1, scale: Optional[float] = None) -> torch.Tensor:
    """out[t] = softmax(q[t] K^T * scale) V over the first ctx_len[t] cached tokens of block-table row bt_row[t]."""
    if not q.is_cuda:
        o = reference.paged_attention(q, kcache, vcache, block_tables, bt_row, ctx_len, n_q, n_kv, hd, scale)
        if out is not None:
            out.copy_(o)
            return out
        return o
    T = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if out is None:
        out = torch.empty(T, n_q * hd, dtype=torch.bfloat16, device=q.device)
    assert block_tables.dtype == torch.int32 and ctx_len.dtype == torch.int32 and block_tables.stride(1) == 1
    ws = None
    if splits > 1:
        need = T * n_q * splits * (hd + 1)
        key = q.device.index or 0
        ws = _attn_ws.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=q.device)
            _attn_ws[key] = ws
    _lib.check(_lib.lib().dmoe_paged_attention(
        _vp(q), c_ll(q.stride(0)), _vp(kcache), _vp(vcache), _vp(block_tables), c_int(block_tables.stride(0)),
        _vp(bt_row), _vp(ctx_len), c_int(kcache.shape[1]), c_int(T), c_int(n_q), c_int(n_kv), c_int(hd),
        c_float(scale), c_int(splits), _vp(out), c_ll(out.stride(0)), _vp(ws), _st()), "dmoe_paged_attention")
    return out


def embed(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not table.is_cuda:
        o = table[ids.long()]
        if out is not None:
            out.copy_(o)
            return out
        return o
    T, (V, H) = ids.shape[0], table.shape
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    assert ids.dtype == torch.int32 and table.dtype == torch.bfloat16 and table.is_contiguous()
    _lib.check(_lib.lib().dmoe_embed(_vp(ids), _vp(table), _vp(out), c_int(T), c_int(H), c_int(V), c_ll(out.stride(0)),
                                     _st()), "dmoe_embed")
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy sampling: int32 ids of the row maxima (first maximum wins)."""
    if not logits.is_cuda:
        o = logits.float().argmax(-1).int()
        if out is not None:
            out.copy_(o)
            return out
        return o
    T, V = logits.shape
    if out is None:
        out = torch.empty(T, dtype=torch.int32, device=logits.device)
    assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    _lib.check(_lib.lib().dmoe_argmax(_vp(logits), c_int(logits.dtype == torch.float32), c_ll(logits.stride(0)),
                                      c_int(T), c_int(V), _vp(out), _st()), "dmoe_argmax")
    return out


def permute_rows(src: torch.Tensor, mapping: torch.Tensor, repeat: int = 1, gather: bool = False,
                 out: Optional[torch.Tensor] = None, n_out: Optional[int] = None) -> torch.Tensor:
    """scatter: out[mapping[i]] = src[i // repeat]; gather: out[i] = src[mapping[i]]. mapping int32, < 0 skipped."""
    n = mapping.numel()
    if not src.is_cuda:
        o = reference.permute_rows(src, mapping, repeat, gather, n_out)
        if out is not None:
            out.copy_(o)
            return out
        return o
    H = src.shape[1]
    if out is None:
        out = torch.zeros(n_out if n_out is not None else n, H, dtype=src.dtype, device=src.device)
    assert mapping.dtype == torch.int32 and src.dtype == torch.bfloat16 and src.stride(1) == 1
    _lib.check(_lib.lib().dmoe_permute_rows(_vp(src), c_ll(src.stride(0)), _vp(out), c_ll(out.stride(0)), _vp(mapping),
                                            c_int(n), c_int(H), c_int(repeat), c_int(int(gather)), _st()),
               "dmoe_permute_rows")
    return out


def gather_ptrs(ptrs: torch.Tensor, n: int, H: int, out: torch.Tensor) -> torch.Tensor:
    """out[i] = the bf16 row of H elements at device address ptrs[i] (int64 device tensor)."""
    assert ptrs.is_cuda and ptrs.dtype == torch.int64
    _lib.check(_lib.lib().dmoe_gather_ptrs(_vp(ptrs), _vp(out), c_ll(out.stride(0)), c_int(n), c_int(H), _st()),
               "dmoe_gather_ptrs")
    return out


def route(x: torch.Tensor, norm_w: Optional[torch.Tensor], eps: float, gate_w: torch.Tensor, top_k: int,
          renormalize: bool = True, y: Optional[torch.Tensor] = None, counts: Optional[torch.Tensor] = None,
          want_logits: bool = False, logit_bias: Optional[torch.Tensor] = None):
    """(RMSNorm ->) gate -> softmax -> top-k. Returns (y, topk_ids int32 [T,k], topk_w fp32 [T,k], logits or None).
    ``counts`` (int32 [E], device) is incremented per routed (token, k) pair. ``logit_bias`` (fp32 [E]) is added to
    the gate logits (synthetic popularity skew)."""
    if not x.is_cuda:
        yy, ids, w, logits = reference.route(x, norm_w, eps, gate_w, top_k, renormalize, logit_bias)
        if counts is not None:
            counts += torch.bincount(ids.reshape(-1).long(), minlength=gate_w.shape[0]).int()
        if y is not None:
            y.copy_(yy)
            yy = y
        return yy, ids, w, (logits if want_logits else None)
    T, H = x.shape
    E = gate_w.shape[0]
    if y is None:
        y = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    ids = torch.empty(T, top_k, dtype=torch.int32, device=x.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=x.device)
    logits = torch.empty(T, E, dtype=torch.float32, device=x.device) if want_logits else None
    assert gate_w.is_contiguous() and gate_w.dtype == torch.bfloat16 and x.stride(1) == 1
    assert logit_bias is None or (logit_bias.dtype == torch.float32 and logit_bias.is_cuda and logit_bias.numel() == E)
    _lib.check(_lib.lib().dmoe_route(
        _vp(x), c_ll(x.stride(0)), _vp(norm_w), c_float(eps), _vp(gate_w), c_int(T), c_int(H), c_int(E), c_int(top_k),
        c_int(int(renormalize)), _vp(y), c_ll(y.stride(0)), _vp(ids), _vp(w), _vp(logits), _vp(counts),
        _vp(logit_bias), _st()), "dmoe_route")
    return y, ids, w, logits


class DispatchBuffers:
    """Device buffers of the local (single GPU) expert dispatch: sorted rows, token records, offsets, scratch."""

    def __init__(self, capacity: int, H: int, E: int, device, dtype=torch.bfloat16):
        self.capacity, self.H, self.E = capacity, H, E
        self.xs = torch.zeros(capacity, H, dtype=dtype, device=device)
        self.recs = torch.zeros(capacity, 4, dtype=torch.int32, device=device)
        self.offs = torch.zeros(E + 1, dtype=torch.int32, device=device)
        self.ws = torch.zeros(2 * E + 8, dtype=torch.int32, device=device)
        self.x_bases = torch.tensor([self.xs.data_ptr()], dtype=torch.int64, device=device)
        self.rec_bases = torch.tensor([self.recs.data_ptr()], dtype=torch.int64, device=device)

    @property
    def counts(self):
        return self.ws[: self.E]


def dispatch_local(y: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, buf: DispatchBuffers) -> None:
    """Copies every routed (token, k) row of y into ``buf.xs`` sorted by expert, writes ``buf.offs`` ([E+1]) and the
    token records ``buf.recs`` = (rank 0, dst row t*k+j, weight bits, expert). ``buf.counts`` must hold the histogram
    produced by :func:`route`; it is cleared for the next layer."""
    T, K = topk_ids.shape
    if not y.is_cuda:
        pos = reference.sort_by_expert(topk_ids).long()
        buf.offs.copy_(reference.expert_offsets(topk_ids, buf.E))
        src = torch.arange(T * K) // K
        buf.xs[pos] = y[src]
        buf.recs[pos, 0] = 0
        buf.recs[pos, 1] = torch.arange(T * K, dtype=torch.int32)
        buf.recs[pos, 2] = topk_w.reshape(-1).contiguous().view(torch.int32)
        buf.recs[pos, 3] = topk_ids.reshape(-1)
        buf.counts.zero_()
        return
    assert T * K <= buf.capacity
    s = scratch(y.device)
    _lib.check(_lib.lib().dmoe_dispatch_local(
        _vp(y), c_ll(y.stride(0)), _vp(topk_ids), _vp(topk_w), c_int(T), c_int(K), c_int(buf.H), c_int(buf.E),
        c_int(buf.E), c_int(0), _vp(buf.ws), _vp(buf.offs), _vp(buf.x_bases), c_ll(buf.xs.stride(0)),
        _vp(buf.rec_bases), c_int(buf.capacity), _vp(s.status), _st()), "dmoe_dispatch_local")


# ---- fused attention-side senders (csrc/kernels/sender.cu); CUDA only -------------------------------------------------
def norm_gather(resid: Optional[torch.Tensor], add: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                resid_out: Optional[torch.Tensor], dst_ptrs: torch.Tensor, n_dst: int, dst_row0: int, ld_dst: int,
                T: int, H: int, wait_flags: Optional[torch.Tensor] = None, n_wait: int = 0,
                wait_epoch: Optional[torch.Tensor] = None, signal_ptrs: Optional[torch.Tensor] = None,
                n_signal: int = 0, signal_slot: int = 0, signal_epoch: Optional[torch.Tensor] = None,
                ticket: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """[wait for ``wait_flags``] resid_out = resid + add.sum(1); rmsnorm(resid_out) * w is stored to rows
    [dst_row0, dst_row0 + T) of every buffer named in ``dst_ptrs`` (int64 device tensor of n_dst addresses, peers
    included); then the flags in ``signal_ptrs`` are released. ``add`` is [T, P, H] (or [T, H]) bf16."""
    d = _lib.DmoeNormGather()
    if add is not None and add.dim() == 2:
        add = add.unsqueeze(1)
    d.resid_in, d.add, d.w, d.resid_out = _lib.ptr(resid), _lib.ptr(add), w.data_ptr(), _lib.ptr(resid_out)
    d.dst_ptrs, d.n_dst, d.dst_row0, d.ld_dst = dst_ptrs.data_ptr(), n_dst, dst_row0, ld_dst
    d.ld_in = resid.stride(0) if resid is not None else 0
    d.ld_out = resid_out.stride(0) if resid_out is not None else 0
    d.n_add = 0 if add is None else add.shape[1]
    d.add_row_stride = add.stride(0) if add is not None else 0
    d.add_part_stride = add.stride(1) if add is not None else 0
    d.eps, d.T, d.H = eps, T, H
    d.wait_flags, d.n_wait, d.wait_epoch = _lib.ptr(wait_flags), n_wait, _lib.ptr(wait_epoch)
    d.signal_ptrs, d.n_signal, d.signal_slot = _lib.ptr(signal_ptrs), n_signal, signal_slot
    d.signal_epoch, d.ticket, d.status = _lib.ptr(signal_epoch), _lib.ptr(ticket), _lib.ptr(status)
    _lib.check(_lib.lib().dmoe_norm_gather(ctypes.byref(d), _st()), "dmoe_norm_gather")


def route_dispatch(resid: torch.Tensor, norm_w: torch.Tensor, eps: float, gate_w: Optional[torch.Tensor], top_k: int,
                   renormalize: bool, T: int, *, add: Optional[torch.Tensor] = None, n_add: int = 0,
                   add_slot_stride: int = 0, ld_add: int = 0, y: Optional[torch.Tensor] = None,
                   topk_ids: Optional[torch.Tensor] = None, topk_w: Optional[torch.Tensor] = None,
                   logit_bias: Optional[torch.Tensor] = None, x_bases=None, rec_bases=None, cnt_bases=None,
                   flag_bases=None, ld_dst: int = 0, experts_per_rank: int = 1, n_dst: int = 0, my_rank: int = 0,
                   ret_rank: Optional[int] = None,
                   region_cap: int = 0, disp_epoch=None, wait_flags=None, n_wait: int = 0, wait_epoch=None, ticket=None,
                   status=None) -> None:
    """One launch for the post-attention half of a layer on an attention GPU: [wait for the TP peers' o_proj flags]
    resid[:T] += the ``n_add`` partial-row slots of ``add``; RMSNorm; gate; softmax; top-k; dispatch of every routed row
    into its expert's receive region on the owning GPU (peer stores) with a release flag per expert GPU."""
    H = resid.shape[1]
    d = _lib.DmoeRouteDispatch()
    d.resid, d.ld_resid, d.add, d.n_add = resid.data_ptr(), resid.stride(0), _lib.ptr(add), n_add
    d.add_slot_stride, d.ld_add = add_slot_stride, ld_add
    d.norm_w, d.eps, d.gate_w, d.logit_bias = norm_w.data_ptr(), eps, _lib.ptr(gate_w), _lib.ptr(logit_bias)
    d.T, d.H, d.E, d.K, d.renorm = T, H, (gate_w.shape[0] if gate_w is not None else 0), top_k, int(renormalize)
    d.y, d.ld_y = _lib.ptr(y), (y.stride(0) if y is not None else 0)
    d.topk_ids, d.topk_w = _lib.ptr(topk_ids), _lib.ptr(topk_w)
    d.x_bases, d.rec_bases, d.cnt_bases, d.flag_bases = (_lib.ptr(t) for t in (x_bases, rec_bases, cnt_bases, flag_bases))
    d.ld_dst, d.experts_per_rank, d.n_dst, d.my_rank, d.region_cap = ld_dst, experts_per_rank, n_dst, my_rank, region_cap
    d.ret_rank, d.ret_rank_set = (ret_rank, 1) if ret_rank is not None else (0, 0)
    d.disp_epoch, d.wait_flags, d.n_wait, d.wait_epoch = _lib.ptr(disp_epoch), _lib.ptr(wait_flags), n_wait, _lib.ptr(wait_epoch)
    d.ticket, d.status = _lib.ptr(ticket), _lib.ptr(status)
    _lib.check(_lib.lib().dmoe_route_dispatch(ctypes.byref(d), _st()), "dmoe_route_dispatch")


def ids_gather(src: torch.Tensor, n: int, dst_ptrs: torch.Tensor, n_dst: int, dst0: int,
               signal_ptrs: Optional[torch.Tensor] = None, signal_slot: int = 0,
               signal_epoch: Optional[torch.Tensor] = None) -> None:
    """The first n int32 of ``src`` are stored at offset dst0 of every buffer in ``dst_ptrs``; then one flag per
    destination is released (the all-gather of a TP group's sampled ids)."""
    _lib.check(_lib.lib().dmoe_ids_gather(_vp(src), c_int(n), _vp(dst_ptrs), c_int(n_dst), c_int(dst0), _vp(signal_ptrs),
                                          c_int(signal_slot), _vp(signal_epoch), _st()), "dmoe_ids_gather")


def wait_flags(flags: torch.Tensor, n: int, epoch: torch.Tensor, status: Optional[torch.Tensor]) -> None:
    """Stand-alone bounded wait: flags[i] >= epoch + 1 for i < n; advances the device-resident epoch."""
    _lib.check(_lib.lib().dmoe_wait_flags(_vp(flags), c_int(n), _vp(epoch), _vp(status), _st()), "dmoe_wait_flags")


# ---- tiled causal attention for prompt tokens (csrc/kernels/attention.cu: prefill_attn_kernel) -----------------------
def prefill_tile_tokens(n_q: int, n_kv: int) -> int:
    """Prompt tokens per tile of :func:`prefill_attention` (64 query rows = tokens x query heads per kv head)."""
    gq = n_q // n_kv
    return 64 // gq if n_q % n_kv == 0 and gq in (1, 2, 4, 8) else 0


def build_prefill_tiles(bt_row, positions, tile_tokens: int, min_len: int = 8):
    """Finds the prompt segments of a flat token batch on the host and cuts them into attention tiles.

    bt_row / positions: int sequences (lists, numpy arrays or CPU tensors) of the batch's rows. A segment is a run of
    consecutive rows of one sequence (same block-table row) at consecutive positions; runs of at least ``min_len``
    rows go to the tiled kernel. Returns (tiles int32 CPU tensor [n, 4] = (first row, tokens, block-table row, first
    position), covered bool CPU tensor [T]): rows not covered stay with the per-token kernel."""
    import numpy as np
    rows = np.asarray(bt_row, dtype=np.int64)
    pos = np.asarray(positions, dtype=np.int64)
    T = len(rows)
    covered = np.zeros(T, dtype=bool)
    tiles = []
    if T == 0 or tile_tokens <= 0:
        return torch.zeros(0, 4, dtype=torch.int32), torch.from_numpy(covered)
    brk = np.nonzero((rows[1:] != rows[:-1]) | (pos[1:] != pos[:-1] + 1))[0] + 1
    starts = np.concatenate([[0], brk])
    ends = np.concatenate([brk, [T]])
    for a, b in zip(starts.tolist(), ends.tolist()):
        if b - a < min_len:
            continue
        covered[a:b] = True
        for t0 in range(a, b, tile_tokens):
            tiles.append((t0, min(tile_tokens, b - t0), int(rows[a]), int(pos[t0])))
    t = torch.tensor(tiles, dtype=torch.int32).reshape(-1, 4)
    return t, torch.from_numpy(covered)


def prefill_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                      tiles: torch.Tensor, n_tiles: int, n_q: int, n_kv: int, hd: int, out: torch.Tensor,
                      scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention of the prompt tokens named by ``tiles`` (device int32 [>= n_tiles, 4], see
    :func:`build_prefill_tiles`) over the paged cache, which already holds their own K / V; writes their rows of
    ``out``. Every tile streams its sequence's K / V once (the per-token kernel streams it once per row)."""
    if n_tiles == 0:
        return out
    assert q.is_cuda and tiles.is_cuda and tiles.dtype == torch.int32 and tiles.is_contiguous()
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    _lib.check(_lib.lib().dmoe_prefill_attention(
        _vp(q), c_ll(q.stride(0)), _vp(kcache), _vp(vcache), _vp(block_tables), c_int(block_tables.stride(0)), _vp(tiles),
        c_int(n_tiles), c_int(kcache.shape[1]), c_int(n_q), c_int(n_kv), c_int(hd), c_float(scale), _vp(out),
        c_ll(out.stride(0)), _st()), "dmoe_prefill_attention")
    return out
