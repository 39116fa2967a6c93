"""bf16 GEMMs on the tcgen05 kernel of ``csrc/kernels/gemm.cu``.

``linear``          y = x @ w.T (+ residual)                         -- reference: disagmoe/models/linear.py:131-136
``grouped_swiglu``  act = silu(x @ w13[g][:I].T) * (x @ w13[g][I:].T)   -- reference: disagmoe/models/experts.py:84-88
``grouped_linear``  y = x @ w2[g].T per expert group                   -- reference: disagmoe/models/experts.py:89
``grouped_combine`` the same GEMM whose epilogue scales each row by its router weight and scatters it to the
                    row (and GPU) it came from                         -- reference: disagmoe/frontend/engine.py:731-734

Weights are K-contiguous ``[groups, out, in]``. CPU tensors take a plain PyTorch path (used by the fp32 CPU
configuration and as the numerical reference); CUDA tensors always run the sm_100a kernel.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib

EPI_PLAIN, EPI_SWIGLU, EPI_COMBINE = 0, 1, 2
STREAM_K = True      # default work distribution of every GEMM launched without an explicit split (tests may turn it off)
TRACE = None         # profiling aid: an int64 [8] CUDA tensor that CTA 0 of every launch fills with nanosecond stamps
_num_sms_cache = {}


def num_sms(device=None) -> int:
    """SM count of a CUDA device (read once per device)."""
    idx = torch.device(device).index if device is not None else None
    if idx is None:
        idx = torch.cuda.current_device() if torch.cuda.is_available() else -1
    if idx not in _num_sms_cache:
        _num_sms_cache[idx] = torch.cuda.get_device_properties(idx).multi_processor_count if idx >= 0 else 148
    return _num_sms_cache[idx]


class _Scratch:
    """Per-device split-K workspace, tile counters and status word (allocated once, reused by every call)."""

    def __init__(self, device):
        self.device = device
        self.ws = torch.empty(64 << 20, dtype=torch.uint8, device=device)
        self.counters = torch.zeros(65536, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def ensure(self, nbytes):
        if nbytes > self.ws.numel():
            self.ws = torch.empty(int(nbytes * 1.25), dtype=torch.uint8, device=self.device)


_scratch = {}


def scratch(device) -> _Scratch:
    key = torch.device(device).index or 0
    if key not in _scratch:
        _scratch[key] = _Scratch(torch.device("cuda", key))
    return _scratch[key]


def check_status(device=None) -> int:
    """Reads (and clears) the device status word; non-zero means a kernel gave up on a bounded wait."""
    s = scratch(device if device is not None else torch.cuda.current_device())
    v = int(s.status.item())
    if v != 0:
        s.status.zero_()
    return v


def pick_splitk(T: int, F: int, K: int, bn: int, sms: int = 0) -> int:
    """Split-K factor of a dense GEMM: enough (tile, split) work items to occupy most of the SMs when the output
    has few tiles (decode-size token counts), never more than one split per 4 K-blocks."""
    sms = sms or num_sms()
    tiles = ((F + 127) // 128) * ((T + bn - 1) // bn)
    kblocks = (K + 63) // 64
    if tiles >= sms * 80 // 148 or kblocks < 8:
        return 1
    return max(1, min((sms * 128 // 148 + tiles // 2) // tiles, kblocks // 4, 16))


def pick_dense(T: int, F: int, K: int, sms: int = 0):
    """(token tile, split-K factor) of a dense GEMM below one wave of tiles, by a cost model fitted to the tile /
    split sweep of benchmark/ops/dense_gemm.py on B200. At these sizes a CTA is bound by what its SM can pull from L2
    (~100 GB/s: 16 KB of weights plus bn x 128 B of tokens per K block), so the model counts, per CTA, the bytes of
    its K range times the number of waves, the parked and re-read partial tiles of a split (the last arriver reads
    them chunk by chunk, latency-bound) and a fixed launch + pipeline-fill cost. It reproduces the order of the
    measured configurations (QKV and o_proj of Mixtral at 64-512 tokens)."""
    sms = sms or num_sms()
    kblocks = (K + 63) // 64
    mt = (F + 127) // 128
    best = None
    for bn in (32, 64, 128, 256):
        if bn < 32 or (bn > 32 and bn // 2 >= T):
            continue                      # a tile twice as wide as the batch only adds shared-memory traffic
        nt = (T + bn - 1) // bn
        for sk in (1, 2, 3, 4, 6, 8):
            per = (kblocks + sk - 1) // sk
            if sk > 1 and (per < 8 or (kblocks + per - 1) // per != sk):
                continue
            units = mt * nt * sk
            if sk > 1 and units > sms:
                continue                  # a split that spills into a second wave measured far slower than whole tiles
            waves = (units + sms - 1) // sms
            cost = 6.0 + waves * per * (16384 + bn * 128) / 1e5 + (bn // 32) * 0.3
            if sk > 1:
                cost += 128 * bn * 4 / 1e5 + (bn // 32) * sk * 0.35
            if best is None or cost < best[0] - 1e-9:
                best = (cost, bn, sk)
    return best[1], best[2]


def pick_bn(tokens_per_group: int, epi: int) -> int:
    cap = 128 if epi == EPI_SWIGLU else 256
    bn = 32
    while bn < tokens_per_group and bn < cap:
        bn *= 2
    return bn


def want_streamk(epi: int, F: int, G: int, T: int, bn: int, sms: int) -> bool:
    """Work distribution of a grouped GEMM, from measurements on B200 (benchmark/ops/grouped_gemm.py): the stream-K
    tail pays off when the expected tile count fills the last wave of CTAs badly (few experts with long K loops, the
    down-projection at decode sizes); the SwiGLU up-projection, whose partial tiles carry two accumulators, is faster
    with whole tiles. Group sizes are only known on the device: the estimate assumes even routing."""
    if not STREAM_K or epi == EPI_SWIGLU:
        return False
    tiles = ((F + 127) // 128) * max(G, (T + bn - 1) // bn)
    waves = (tiles + sms - 1) // sms
    return tiles / (waves * sms) < 0.85


def _group_hint(T: int, G: int) -> int:
    """Token-tile hint for a grouped GEMM whose group sizes are only known on the device: the mean group size plus
    head-room for routing imbalance, so that most groups fit one token tile (a second tile re-reads the weights)."""
    mean = (T + G - 1) // G
    return mean + mean // 2 + 8 if G > 1 else mean


class GemmComm:
    """Multi-GPU hooks of a grouped GEMM launch (see ``DmoeGemm`` in csrc/kernels/dmoe_kernels.h).

    seg_cnt [S, G] int32 (device): rows source s delivered for group g; region s = rows [s*seg_cap, (s+1)*seg_cap).
    wait_flags [n_wait] int32 + wait_epoch [1]: arrival gate. signal_ptrs int64 [n_signal] (peer flag arrays) +
    signal_slot + signal_epoch [1]: completion signal. done_ticket [1]: zero-initialised scratch int.
    """

    def __init__(self, seg_cnt=None, S=0, seg_cap=0, wait_flags=None, n_wait=0, wait_epoch=None, signal_ptrs=None,
                 n_signal=0, signal_slot=0, signal_epoch=None, done_ticket=None, fanout=0, group_regions=False,
                 clear=None, shard_rows=0, rs_bases=None, rs_rows=0, rs_slot=0, rs_cap=0, rope: "Optional[RopeAppend]" = None):
        self.seg_cnt, self.S, self.seg_cap = seg_cnt, S, seg_cap
        self.wait_flags, self.n_wait, self.wait_epoch = wait_flags, n_wait, wait_epoch
        self.signal_ptrs, self.n_signal, self.signal_slot = signal_ptrs, n_signal, signal_slot
        self.signal_epoch, self.done_ticket = signal_epoch, done_ticket
        self.fanout, self.group_regions, self.clear = fanout, group_regions, clear
        # tensor-parallel attention: all-gather prologue (X arrives in shards of shard_rows rows, one wait flag per
        # shard), reduce-scatter epilogue (row t -> rank t // rs_rows, slot rs_slot of its partial buffer)
        self.shard_rows = shard_rows
        self.rs_bases, self.rs_rows, self.rs_slot, self.rs_cap = rs_bases, rs_rows, rs_slot, rs_cap
        self.rope = rope

    def fill(self, d):
        d.seg_cnt, d.S, d.seg_cap = _lib.ptr(self.seg_cnt), self.S, self.seg_cap
        d.wait_flags, d.n_wait, d.wait_epoch = _lib.ptr(self.wait_flags), self.n_wait, _lib.ptr(self.wait_epoch)
        d.signal_ptrs, d.n_signal, d.signal_slot = _lib.ptr(self.signal_ptrs), self.n_signal, self.signal_slot
        d.signal_epoch, d.done_ticket = _lib.ptr(self.signal_epoch), _lib.ptr(self.done_ticket)
        d.fanout = self.fanout
        d.group_regions = int(self.group_regions)
        d.clear_ptr, d.clear_n = _lib.ptr(self.clear), (0 if self.clear is None else self.clear.numel())
        d.shard_rows = self.shard_rows
        d.rs_bases, d.rs_rows, d.rs_slot, d.rs_cap = _lib.ptr(self.rs_bases), self.rs_rows, self.rs_slot, self.rs_cap
        if self.rope is not None:
            r = self.rope
            d.rope_table, d.positions, d.slots = r.table.data_ptr(), r.positions.data_ptr(), _lib.ptr(r.slots)
            d.kcache, d.vcache = r.kcache.data_ptr(), r.vcache.data_ptr()
            d.n_q, d.n_kv, d.hd, d.rope_max_pos = r.n_q, r.n_kv, r.hd, r.table.shape[0]


class RopeAppend:
    """QKV epilogue: neox RoPE on the q / k heads and K / V append to the paged cache (see ``DmoeGemm``).

    table: fp32 [max_pos, hd / 2, 2] from :func:`rope_table`; positions int32 [T]; slots int64 [T] or None;
    kcache / vcache [blocks, block_size, n_kv, hd] bf16."""

    def __init__(self, table, positions, slots, kcache, vcache, n_q, n_kv, hd):
        assert table.dtype == torch.float32 and table.is_contiguous() and table.shape[1] == hd // 2
        assert positions.dtype == torch.int32 and (slots is None or slots.dtype == torch.int64)
        assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == torch.bfloat16
        self.table, self.positions, self.slots, self.kcache, self.vcache = table, positions, slots, kcache, vcache
        self.n_q, self.n_kv, self.hd = n_q, n_kv, hd


_rope_tables = {}


def rope_table(max_pos: int, hd: int, theta: float, device) -> torch.Tensor:
    """fp32 [max_pos, hd / 2, 2] = (cos, sin)(pos * theta^(-2 d / hd)), computed on the device with the arithmetic
    of the stand-alone RoPE kernel; cached per (device, max_pos, hd, theta)."""
    device = torch.device(device)
    key = (device.index or 0, max_pos, hd, float(theta))
    t = _rope_tables.get(key)
    if t is None:
        t = torch.empty(max_pos, hd // 2, 2, dtype=torch.float32, device=device)
        with torch.cuda.device(device):
            _lib.check(_lib.lib().dmoe_rope_table(ctypes.c_void_p(t.data_ptr()), ctypes.c_int(max_pos), ctypes.c_int(hd),
                                                  ctypes.c_float(theta), ctypes.c_void_p(_lib.stream_ptr())),
                       "dmoe_rope_table")
        _rope_tables[key] = t
    return t


def _launch(W, X, Y, R, offs, recs, bases, G, T, F, K, epi, bn, splitk, ldy, y_f32, comm: Optional[GemmComm] = None,
            streamk: bool = False, pair: bool = False, w_blocked: bool = False):
    s = scratch(X.device)
    d = _lib.DmoeGemm()
    d.w_blocked = int(w_blocked)
    d.trace = TRACE.data_ptr() if TRACE is not None else None
    d.streamk, d.n_counters = int(streamk and splitk <= 1 and not pair), s.counters.numel()
    d.pair = int(pair)
    d.combine_vec = int(epi == EPI_COMBINE and F % 8 == 0 and ldy % 8 == 0 and _bases_aligned(bases))
    if comm is not None:
        comm.fill(d)
    d.W, d.X, d.Y, d.R = W.data_ptr(), X.data_ptr(), _lib.ptr(Y), _lib.ptr(R)
    d.offs, d.recs, d.bases = _lib.ptr(offs), _lib.ptr(recs), _lib.ptr(bases)
    if splitk > 1:
        need = _lib.lib().dmoe_gemm_workspace_bytes(T, F, bn, splitk)
        s.ensure(need)
    d.ws, d.counters, d.status = s.ws.data_ptr(), s.counters.data_ptr(), s.status.data_ptr()
    d.ws_bytes = s.ws.numel()
    d.ldx = X.stride(0)
    d.ldy = ldy
    d.ldr = R.stride(0) if R is not None else 0
    d.G, d.T, d.F, d.K = G, T, F, K
    d.epi, d.bn, d.splitk, d.y_f32 = epi, bn, splitk, int(y_f32)
    _lib.check(_lib.lib().dmoe_gemm(ctypes.byref(d), _lib.stream_ptr()), "dmoe_gemm")


def _check_x(x):
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype == torch.bfloat16, "x must be [T, K] bf16, K contiguous"
    assert x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0, "x rows must be 16-byte aligned"


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, bn: int = 0,
           splitk: int = 0, comm: Optional["GemmComm"] = None, pair: bool = False) -> torch.Tensor:
    """y[T, F] = x[T, K] @ w[F, K].T (+ residual[T, F]). ``pair``: CTA pairs (tcgen05 cta_group::2) on tiles of 256
    weight rows x ``bn`` (128 / 256) tokens, whole tiles."""
    T, K = x.shape
    F = w.shape[0]
    if not x.is_cuda:
        y = torch.nn.functional.linear(x.float(), w.float())
        if residual is not None:
            y = y + residual.float()
        y = y.to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_x(x)
    assert w.is_contiguous() and w.dtype == torch.bfloat16 and w.shape[1] == K
    odt = out_dtype or torch.bfloat16
    scatter = comm is not None and comm.rs_bases is not None      # reduce-scatter epilogue: rows go to the peers
    if out is None and not scatter:
        out = torch.empty(T, F, dtype=odt, device=x.device)
    assert scatter or (out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32))
    if T == 0:
        return out
    # splitk = 0 (default): with at least one full wave of tiles, whole tiles per CTA plus a stream-K tail (the tiles of
    # the last, partial wave are cut along K into equal shares for all SMs); with fewer tiles than SMs (decode sizes)
    # plain split-K with a factor that fills the SMs. An explicit splitk >= 1 selects split-K with that factor.
    sms = num_sms(x.device)
    auto_sk = 0
    if not bn:
        bn = pick_bn(T, EPI_PLAIN)
        if ((F + 127) // 128) * ((T + bn - 1) // bn) < sms and not pair:
            bn, auto_sk = pick_dense(T, F, K, sms)
    if pair:
        bn = 256 if bn not in (128, 256) else bn
        splitk = 1
    streamk = splitk == 0 and STREAM_K and ((F + 127) // 128) * ((T + bn - 1) // bn) >= sms
    if streamk:
        splitk = 1
    else:
        splitk = splitk or auto_sk or pick_splitk(T, F, K, bn, sms)
    _launch(w, x, out, residual, None, None, None, 1, T, F, K, EPI_PLAIN, bn, splitk,
            F if scatter else out.stride(0), (not scatter) and out.dtype == torch.float32, comm, streamk=streamk,
            pair=pair)
    return out


def _grouped_ref(x, w, offs, swiglu):
    offs = offs.tolist()
    G = w.shape[0]
    F = w.shape[1] // 2 if swiglu else w.shape[1]
    y = torch.zeros(x.shape[0], F, dtype=torch.float32, device=x.device)
    for g in range(G):
        a, b = offs[g], offs[g + 1]
        if b <= a:
            continue
        h = x[a:b].float() @ w[g].float().T
        if swiglu:
            h = torch.nn.functional.silu(h[:, :F]) * h[:, F:]
        y[a:b] = h
    return y


def grouped_swiglu(x: torch.Tensor, w13: torch.Tensor, offs: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
                   bn: int = 0, comm: Optional[GemmComm] = None, streamk: Optional[bool] = None,
                   pair: bool = False, w_blocked: bool = False) -> torch.Tensor:
    """act[T, I] = silu(x @ w13[g, :I].T) * (x @ w13[g, I:].T) for the rows of group g; w13 is [G, 2I, K]."""
    T, K = x.shape
    G, F2, _ = w13.shape
    I = F2 // 2
    if not x.is_cuda:
        y = _grouped_ref(x, w13, offs, True).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_x(x)
    assert w13.is_contiguous() and w13.dtype == torch.bfloat16
    assert comm is not None or (offs.dtype == torch.int32 and offs.is_cuda)
    if out is None:
        out = torch.empty(T, I, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return out
    bn = bn or (pick_bn(_group_hint(T, G), EPI_COMBINE) if pair else pick_bn(_group_hint(T, G), EPI_SWIGLU))
    if pair:
        bn = max(bn, 128)
    sk = want_streamk(EPI_SWIGLU, I, G, T, bn, num_sms(x.device)) if streamk is None else streamk
    _launch(w13, x, out, None, offs, None, None, G, T, I, K, EPI_SWIGLU, bn, 1, out.stride(0), False, comm,
            streamk=sk, pair=pair, w_blocked=w_blocked)
    return out


def grouped_linear(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, out: Optional[torch.Tensor] = None,
                   bn: int = 0, streamk: Optional[bool] = None, pair: bool = False,
                   w_blocked: bool = False) -> torch.Tensor:
    """y[T, F] = x @ w[g].T for the rows of group g; w is [G, F, K]."""
    T, K = x.shape
    G, F, _ = w.shape
    if not x.is_cuda:
        y = _grouped_ref(x, w, offs, False).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_x(x)
    assert w.is_contiguous() and w.dtype == torch.bfloat16 and offs.dtype == torch.int32 and offs.is_cuda
    if out is None:
        out = torch.empty(T, F, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return out
    bn = bn or pick_bn(_group_hint(T, G), EPI_PLAIN)
    if pair:
        bn = max(bn, 128)
    sk = want_streamk(EPI_PLAIN, F, G, T, bn, num_sms(x.device)) if streamk is None else streamk
    _launch(w, x, out, None, offs, None, None, G, T, F, K, EPI_PLAIN, bn, 1, out.stride(0), False, streamk=sk, pair=pair,
            w_blocked=w_blocked)
    return out


def block_weight(w: torch.Tensor) -> torch.Tensor:
    """Re-orders a K-contiguous weight stack [G, R, K] (or [R, K]) tile by tile: [G, R / 128, K / 64, 128, 64], returned
    with the ORIGINAL shape (only the memory order changes), for launches with ``w_blocked=True``. Every 128-row x
    64-column box the GEMM fetches is then 16 KB of consecutive addresses instead of 128 runs of 128 bytes one weight
    row apart. R must be a multiple of 128 (for SwiGLU stacks: the gate and the up half each) and K of 64."""
    shape = w.shape
    w3 = w if w.dim() == 3 else w.unsqueeze(0)
    G, R, K = w3.shape
    assert R % 128 == 0 and K % 64 == 0, "blocked weights need whole 128 x 64 tiles"
    return w3.view(G, R // 128, 128, K // 64, 64).permute(0, 1, 3, 2, 4).contiguous().view(shape)


def unblock_weight(w: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`block_weight`: a row-major copy of a tile-blocked stack."""
    shape = w.shape
    w3 = w if w.dim() == 3 else w.unsqueeze(0)
    G, R, K = w3.shape
    return w3.view(G, R // 128, K // 64, 128, 64).permute(0, 1, 3, 2, 4).contiguous().view(shape)


_bases_checked = {}


def _bases_aligned(bases: torch.Tensor) -> bool:
    """Are all destination pointers of a combine table 16-byte aligned? Read back once per table (tables are built at
    start-up and never change); a table first seen during a graph capture, where nothing can be read back, counts as
    unaligned and keeps the 2-byte stores."""
    key = (bases.data_ptr(), bases.numel())
    if key not in _bases_checked:
        if torch.cuda.is_current_stream_capturing():
            return False
        _bases_checked[key] = bool((bases % 16 == 0).all().item())
    return _bases_checked[key]


def grouped_combine(x: torch.Tensor, w: torch.Tensor, offs: Optional[torch.Tensor], recs: torch.Tensor,
                    bases: torch.Tensor, ld_out: int, bn: int = 0, outs=None, comm: Optional[GemmComm] = None,
                    streamk: Optional[bool] = None, pair: bool = False, w_blocked: bool = False) -> None:
    """GEMM-2 with the combine epilogue: row t of group g becomes ``weight[t] * (x[t] @ w[g].T)`` written to row
    ``recs[t, 1]`` of the buffer ``bases[recs[t, 0]]`` (row stride ``ld_out`` elements).

    recs: int32 [T, 4] = (dst_rank, dst_row or -1, weight as fp32 bits, 0). bases: int64 [n_ranks] device
    tensor of raw pointers (peer buffers included). ``outs`` (CPU path only) is the list of destination tensors.
    """
    T, K = x.shape
    G, F, _ = w.shape
    if not x.is_cuda:
        y = _grouped_ref(x, w, offs, False)
        wts = recs[:, 2].contiguous().view(torch.float32)
        for t in range(T):
            r, row = int(recs[t, 0]), int(recs[t, 1])
            if row >= 0:
                outs[r][row] = (y[t] * wts[t]).to(outs[r].dtype)
        return
    _check_x(x)
    assert recs.dtype == torch.int32 and recs.is_contiguous() and recs.shape[1] == 4 and bases.dtype == torch.int64
    if T == 0:
        return
    bn = bn or pick_bn(_group_hint(T, G), EPI_COMBINE)
    if pair:
        bn = max(bn, 128)
    sk = want_streamk(EPI_COMBINE, F, G, T, bn, num_sms(x.device)) if streamk is None else streamk
    _launch(w, x, None, None, offs, recs, bases, G, T, F, K, EPI_COMBINE, bn, 1, ld_out, False, comm, streamk=sk,
            pair=pair, w_blocked=w_blocked)


def swiglu_linear(x: torch.Tensor, w13: torch.Tensor, out: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
    """Dense SwiGLU up-projection: silu(x @ w13[:I].T) * (x @ w13[I:].T); w13 is [2I, K] (a one-group grouped_swiglu)."""
    T, K = x.shape
    I = w13.shape[0] // 2
    if not x.is_cuda:
        h = x.float() @ w13.float().T
        y = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check_x(x)
    assert w13.is_contiguous() and w13.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(T, I, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return out
    bn = bn or pick_bn(T, EPI_SWIGLU)
    _launch(w13, x, out, None, None, None, None, 1, T, I, K, EPI_SWIGLU, bn, 1, out.stride(0), False)
    return out
