"""Device-driven disaggregated decode: attention GPUs and expert GPUs exchange tokens through peer memory.

Ranks [0, A) are attention GPUs, in groups of ``tp`` consecutive ranks that share their sequences (tensor parallel:
heads and KV cache split over the group, residual stream sharded by rows) — groups are data-parallel replicas of
one another; ranks [A, A + X) hold the routed experts (expert parallel, ``num_experts / X`` experts each). One decode
iteration of a micro-batch is, per layer:

    attention rank   [wait combine flags] add+RMSNorm (+ all-gather push) -> QKV (+ RoPE, KV append) -> paged attention
                     -> o_proj (+ residual, or + reduce-scatter push) -> [wait o_proj flags] reduce + RMSNorm + gate +
                     top-k + dispatch: every routed row reserves a slot in its expert's region on the owning expert GPU
                     (one system-scope atomic), then row, record and finally a release flag are stored there
    expert rank      grouped GEMM-1 (+SwiGLU), gated on the arrival flags, reads the rows where they landed
                     -> grouped GEMM-2 whose epilogue scales by the router weight and stores every row into the
                     partial-output buffer of the attention GPU that owns the row, then signals that GPU

Nothing in this chain returns to the host: flags carry device-resident epoch counters, so the whole iteration of a
rank is one CUDA graph. Every attention rank runs two micro-batches through the layers in lock-step order
(mb0, mb1 per layer), so the expert GPUs work on one micro-batch while the attention GPUs work on the other: the
overlap DisagMoE gets from asynchronous layer-wise scheduling (csrc/engine/scheduler.cpp) is obtained here from a
fixed interleaving that needs no scheduler on the critical path.

Reference data path replaced: disagmoe/frontend/engine.py:614-754, csrc/muhelper/muhelper.cpp:189-323,485-515.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import disagmoe_c as C
from ..config import ModelConfig
from ..models import weights as W
from ..models.attention import AttnMeta, MoEAttention
from ..models.experts import MoEExperts
from ..ops import _lib
from ..ops import functional as F
from ..ops import gemm
from .peer import ArenaLayout, PeerArena

c_int, c_ll, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p


def _vp(t):
    return c_vp(0 if t is None else t.data_ptr())


@dataclass
class DisaggShape:
    n_attn: int
    n_expert: int
    n_mb: int           # micro-batches per attention rank
    batch: int          # token rows per micro-batch of one attention group (a TP group shares them)
    top_k: int
    hidden: int
    num_experts: int
    tp: int = 1         # attention tensor-parallel degree: consecutive groups of `tp` attention ranks share sequences
    # layer striping (the reference's step_attn placement, disagmoe/utils/placement.py:369-434): with stripes > 1 the
    # n_attn = stripes attention GPUs form ONE pipeline over the layers instead of data-parallel replicas. Rank g owns
    # a contiguous block of layers and the KV cache of those layers for every micro-batch of the job; the residual
    # stream of a micro-batch is handed from rank g to rank g + 1 by peer stores, and the experts return the output of
    # a stripe's last layer to the rank that owns the next layer.
    stripes: int = 1
    num_layers: int = 0   # needed with stripes > 1 only

    def __post_init__(self):
        if self.stripes > 1:
            assert self.tp == 1 and self.stripes == self.n_attn and self.num_layers >= self.stripes, \
                "layer striping: one pipeline over all attention GPUs, no TP inside a stage, at least one layer each"

    def layers_per_stripe(self) -> int:
        return (self.num_layers + self.stripes - 1) // self.stripes

    def layer_owner(self, l: int) -> int:
        """Attention rank that runs layer l (and the LM head for l == num_layers); -1 without striping."""
        if self.stripes <= 1:
            return -1
        return min(l // self.layers_per_stripe(), self.stripes - 1)

    @property
    def experts_per_rank(self) -> int:
        # experts are dealt out in contiguous blocks of ceil(E / X); the last expert rank may hold fewer
        return (self.num_experts + self.n_expert - 1) // self.n_expert

    @property
    def rows_cap(self) -> int:
        """Rows of the residual stream one attention rank owns at full batch (the sequence shard of a TP rank)."""
        return (self.batch + self.tp - 1) // self.tp

    @property
    def region_cap(self) -> int:   # rows of one expert's receive region: every sender could route all its pairs to it
        return self.n_attn * self.rows_cap * self.top_k


def shard_rows(T: int, tp: int) -> int:
    """Rows per TP rank when T rows are split over tp ranks: rank r owns [r * per, min(T, (r + 1) * per))."""
    return max(1, (T + tp - 1) // tp)


def build_layout(s: DisaggShape) -> ArenaLayout:
    L = ArenaLayout()
    rows = s.experts_per_rank * s.region_cap
    for m in range(s.n_mb):
        L.add(f"recv_rows{m}", rows * s.hidden * 2)
        L.add(f"recv_recs{m}", rows * 16)
        L.add(f"recv_cnt{m}", s.experts_per_rank * 4)      # per-expert row cursors, advanced by the senders
        L.add(f"disp_flag{m}", s.n_attn * 4)
        L.add(f"parts{m}", s.rows_cap * s.top_k * s.hidden * 2)
        L.add(f"comb_flag{m}", s.n_expert * 4)
        if s.stripes > 1:
            # pipeline hand-off: the residual rows of the micro-batch live in the arena so that the previous stage can
            # store them here, and one flag says that they have arrived
            L.add(f"ho_resid{m}", s.rows_cap * s.hidden * 2)
            L.add(f"ho_flag{m}", 4)
        if s.tp > 1:
            # all-gather target: the normalised rows of the whole group, every rank pushes its shard to every member
            L.add(f"hs{m}", s.batch * s.hidden * 2)
            L.add(f"hsflag{m}", s.tp * 4)
            # reduce-scatter target: slot p holds TP rank p's o_proj partial sums of THIS rank's rows. One buffer is
            # enough: a peer writes layer l + 1's partials only after its QKV GEMM saw this rank's layer l + 1 shard,
            # which this rank pushes after it has consumed layer l's partials
            L.add(f"opart{m}", s.tp * s.rows_cap * s.hidden * 2)
            L.add(f"oflag{m}", s.tp * 4)
            L.add(f"nid{m}", s.batch * 4)                  # sampled ids of the whole group
            L.add(f"nidflag{m}", s.tp * 4)
    return L


class AttentionRank:
    """All attention layers + embedding + LM head of one attention GPU, with its KV cache and micro-batch buffers.

    Per layer and micro-batch this rank launches five kernels (six when the attention runs split-KV):

        norm_gather      [wait: experts' combine flags] resid += expert partials; pre-norm; the normalised rows go
                         to the QKV staging buffer of every member of the TP group (all-gather by peer stores)
        QKV GEMM         tcgen05; token tiles gated shard by shard on the members' flags (all-gather prologue);
                         epilogue rotates q / k (RoPE) and appends K / V to the paged cache
        paged attention  this rank's heads, all rows of the group
        o_proj GEMM      tcgen05; with TP the epilogue scatters every row's partial sum to the rank that owns the row
                         (reduce-scatter by peer stores) and signals; without TP it adds the residual in place
        route_dispatch   [wait: members' o_proj flags] ordered sum of the partials + residual; post-norm; gate; top-k;
                         row reservation on the expert GPUs; remote stores of rows + records; release flags

    With tensor parallelism the residual stream is sharded by rows: rank r of a group owns rows [r * per, (r + 1) *
    per) of the group's micro-batch (per = ceil(T / tp)), runs both norms, the router, the dispatch, shared experts /
    dense FFN and the LM head on those rows only, and receives the experts' combine output for those rows only.
    Replaces, for TP groups, the reference's broadcast of inputs (disagmoe/frontend/engine.py:494-535) and its
    all-reduce after o_proj (disagmoe/models/linear.py:1064-1089, csrc/muhelper/comm.cpp:399-416).

    With layer striping (``shape.stripes`` = number of attention ranks) the ranks are the stages of one pipeline over
    the layers: a rank loads the weights and keeps the KV cache of its block of layers only, ``layer`` is a no-op for
    the other layers, the first stage embeds and the last one runs the LM head. After its last layer a stage stores the
    residual rows of the micro-batch into the next stage's residual buffer and releases its hand-off flag; the dispatch
    records of that layer name the next stage as the owner the experts return to."""

    def __init__(self, cfg: ModelConfig, shape: DisaggShape, arena: PeerArena, layout: ArenaLayout, attn_rank: int,
                 num_blocks: int, block_size: int = 16, state_dict: Optional[W.StateDict] = None, device=None):
        self.cfg, self.shape, self.arena, self.layout, self.a = cfg, shape, arena, layout, attn_rank
        dev = device or arena.local.device
        self.device = dev
        dt = torch.bfloat16
        self.tp = shape.tp
        self.tp_rank = attn_rank % shape.tp
        self.group0 = attn_rank // shape.tp * shape.tp      # first attention rank of this TP group
        # layer striping: this rank holds the weights and the KV cache of layers [l0, l1) only
        self.stripes = shape.stripes
        if self.stripes > 1:
            per = shape.layers_per_stripe()
            self.l0 = min(attn_rank * per, cfg.num_layers)
            self.l1 = cfg.num_layers if attn_rank == self.stripes - 1 else min((attn_rank + 1) * per, cfg.num_layers)
        else:
            self.l0, self.l1 = 0, cfg.num_layers
        self.layers: List[Optional[MoEAttention]] = []
        for l in range(cfg.num_layers):
            if not self.l0 <= l < self.l1:
                self.layers.append(None)
                continue
            m = MoEAttention(cfg, l, tp_size=self.tp, tp_rank=self.tp_rank, device=dev, dtype=dt)
            m.load_weights(state_dict) if state_dict is not None else m.init_weights()
            self.layers.append(m)
        names = ["embed_tokens.weight", "norm.weight", "lm_head.weight"]
        sd = state_dict if state_dict is not None else W.init_state_dict(cfg, dev, dt, names)
        self.embed_w = sd["embed_tokens.weight"].to(device=dev, dtype=dt).contiguous()
        self.norm_w = sd["norm.weight"].to(device=dev, dtype=dt)
        self.lm_head_w = sd["lm_head.weight"].to(device=dev, dtype=dt).contiguous()
        S = shape
        B, R, k, H, E = S.batch, S.rows_cap, S.top_k, S.hidden, S.num_experts
        a0 = self.layers[self.l0]
        self.block_size = block_size
        self.max_blocks = (cfg.max_seq_len + block_size - 1) // block_size
        self.kv_cache = torch.zeros(self.l1 - self.l0, 2, num_blocks, block_size, a0.num_kv_heads, cfg.head_dim,
                                    dtype=dt, device=dev)
        self.block_tables = torch.zeros(S.n_mb * B, self.max_blocks, dtype=torch.int32, device=dev)
        self.rope = gemm.rope_table(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta, dev)
        self.qkv_features = a0.q_size + 2 * a0.kv_size
        z = lambda *s, dt_=torch.int32: torch.zeros(*s, dtype=dt_, device=dev)
        self.mb = []
        expert_ranks = [S.n_attn + x for x in range(S.n_expert)]
        group = [self.group0 + i for i in range(self.tp)]
        for m in range(S.n_mb):
            d = dict(
                ids=z(B), positions=z(B), slots=z(B, dt_=torch.int64), ctx_len=z(B), bt_row=z(B),
                resid=torch.zeros(R, H, dtype=dt, device=dev), y=torch.zeros(R, H, dtype=dt, device=dev),
                hfin=torch.zeros(R, H, dtype=dt, device=dev),
                qkv=torch.zeros(B, self.qkv_features, dtype=dt, device=dev),
                attn=torch.zeros(B, a0.q_size, dtype=dt, device=dev),
                disp_epoch=z(1), comb_epoch=z(1), ticket=z(1),
                pre_tiles=z(B, 4), ctx_dec=z(B),
                next_local=z(R), logits=torch.zeros(R, cfg.vocab_size, dtype=torch.float32, device=dev),
                topk_ids=z(R, k), topk_w=torch.zeros(R, k, dtype=torch.float32, device=dev),
                parts=arena.view(layout.offset(f"parts{m}"), (R, k, H), dt),
                comb_flag=arena.view(layout.offset(f"comb_flag{m}"), (S.n_expert,), torch.int32),
                x_bases=arena.ptr_table(expert_ranks, layout.offset(f"recv_rows{m}")),
                rec_bases=arena.ptr_table(expert_ranks, layout.offset(f"recv_recs{m}")),
                cnt_bases=arena.ptr_table(expert_ranks, layout.offset(f"recv_cnt{m}")),
                flag_bases=arena.ptr_table(expert_ranks, layout.offset(f"disp_flag{m}")),
            )
            if self.stripes > 1:
                # the residual rows live in the arena: the previous stage stores them here and releases ho_flag
                nxt = attn_rank + 1 if attn_rank + 1 < self.stripes else attn_rank
                d.update(
                    resid=arena.view(layout.offset(f"ho_resid{m}"), (R, H), dt),
                    ho_flag=arena.view(layout.offset(f"ho_flag{m}"), (1,), torch.int32),
                    ho_next_resid=arena.view(layout.offset(f"ho_resid{m}"), (R, H), dt, rank=nxt),
                    ho_sig_ptrs=arena.ptr_table([nxt], layout.offset(f"ho_flag{m}")),
                    ho_sig_epoch=z(1), ho_wait_epoch=z(1))
            if self.tp > 1:
                d.update(
                    hs=arena.view(layout.offset(f"hs{m}"), (B, H), dt),
                    hs_ptrs=arena.ptr_table(group, layout.offset(f"hs{m}")),
                    hsflag=arena.view(layout.offset(f"hsflag{m}"), (self.tp,), torch.int32),
                    hsflag_ptrs=arena.ptr_table(group, layout.offset(f"hsflag{m}")),
                    opart=arena.view(layout.offset(f"opart{m}"), (self.tp, R, H), dt),
                    opart_ptrs=arena.ptr_table(group, layout.offset(f"opart{m}")),
                    oflag=arena.view(layout.offset(f"oflag{m}"), (self.tp,), torch.int32),
                    oflag_ptrs=arena.ptr_table(group, layout.offset(f"oflag{m}")),
                    next_ids=arena.view(layout.offset(f"nid{m}"), (B,), torch.int32),
                    nid_ptrs=arena.ptr_table(group, layout.offset(f"nid{m}")),
                    nidflag=arena.view(layout.offset(f"nidflag{m}"), (self.tp,), torch.int32),
                    nidflag_ptrs=arena.ptr_table(group, layout.offset(f"nidflag{m}")),
                    hs_sig_epoch=z(1), hs_wait_epoch=z(1), o_sig_epoch=z(1), o_wait_epoch=z(1),
                    nid_sig_epoch=z(1), nid_wait_epoch=z(1), gemm_ticket=z(1))
            else:
                d["hs"] = torch.zeros(B, H, dtype=dt, device=dev)
                d["hs_ptrs"] = torch.tensor([d["hs"].data_ptr()], dtype=torch.int64, device=dev)
                d["next_ids"] = d["next_local"]
            d["hfin_ptrs"] = torch.tensor([d["hfin"].data_ptr()], dtype=torch.int64, device=dev)
            self.mb.append(d)
        self.status = gemm.scratch(dev).status
        self.active = [B] * S.n_mb      # rows of every micro-batch that the next launches process (<= B)
        self.n_pre = [0] * S.n_mb       # prompt tiles of every micro-batch for the tiled causal attention kernel

    def set_active(self, m: int, T: int) -> None:
        """The next launches of micro-batch m process its first T rows (1 <= T <= batch): a serving step fills the
        buffers with however many decode and prompt tokens it scheduled."""
        assert 1 <= T <= self.shape.batch
        self.active[m] = T

    def set_prefill_tiles(self, m: int, bt_row, positions, ctx_len) -> int:
        """Eager (not graph-captured) iterations only: finds the prompt segments among the first ``active`` rows of
        micro-batch m from the host copies of its block-table rows / positions / context lengths and routes them to
        the tiled causal attention kernel; the other rows stay with the per-token kernel. Returns the tile count;
        ``set_prefill_tiles(m, None, None, None)`` switches the tiled kernel off again."""
        if bt_row is None:
            self.n_pre[m] = 0
            return 0
        a0 = self.layers[self.l0]
        tiles, covered = F.build_prefill_tiles(bt_row, positions, F.prefill_tile_tokens(a0.num_heads, a0.num_kv_heads))
        self.n_pre[m] = len(tiles)
        if len(tiles):
            d = self.mb[m]
            d["pre_tiles"][:len(tiles)].copy_(tiles, non_blocking=True)
            cd = torch.as_tensor(ctx_len).clone()
            cd[covered] = 0
            d["ctx_dec"][:len(cd)].copy_(cd, non_blocking=True)
        return len(tiles)

    def rows(self, m: int):
        """(T, rows per TP rank, first own row, one past the last own row) of micro-batch m as currently active."""
        T = self.active[m]
        per = shard_rows(T, self.tp)
        return T, per, min(T, self.tp_rank * per), min(T, (self.tp_rank + 1) * per)

    def _meta(self, m: int) -> AttnMeta:
        d, T = self.mb[m], self.active[m]
        return AttnMeta(d["positions"][:T], d["slots"][:T], self.block_tables, d["bt_row"][:T], d["ctx_len"][:T],
                        max_ctx=self.cfg.max_seq_len)

    def embed(self, m: int) -> None:
        d = self.mb[m]
        _, _, lo, hi = self.rows(m)
        if self.stripes > 1 and self.a != 0:
            return      # the first pipeline stage embeds; the others receive the residual rows by hand-off
        if hi > lo:
            F.embed(d["ids"][lo:hi], self.embed_w, out=d["resid"][:hi - lo])

    def layer(self, l: int, m: int) -> None:
        """Attention half of layer l for micro-batch m, ending with the peer-memory dispatch."""
        if not self.l0 <= l < self.l1:
            return      # another pipeline stage owns this layer
        self.layer_pre(l, m)
        self.layer_attn(l, m)
        self.layer_route_dispatch(l, m)

    def _expert_parts(self, l: int) -> bool:
        """Does layer l start by adding the routed experts' output of layer l - 1? (Not after a dense-FFN layer, which
        sends nothing to the expert GPUs.)"""
        return l > 0 and not self.cfg.is_dense_layer(l - 1)

    def layer_pre(self, l: int, m: int) -> None:
        """[wait for the experts' combine] add + pre-attention RMSNorm on this rank's rows; the normalised rows land in
        the QKV staging buffer of every member of the TP group."""
        d, S, cfg = self.mb[m], self.shape, self.cfg
        T, per, lo, hi = self.rows(m)
        Tm = hi - lo
        a = self.layers[l]
        wait = self._expert_parts(l)
        tp = self.tp
        if self.stripes > 1 and l == self.l0 and self.a > 0:
            # first layer of this stage: the previous stage's residual rows must have landed
            F.wait_flags(d["ho_flag"], 1, d["ho_wait_epoch"], self.status)
        F.norm_gather(d["resid"][:Tm], d["parts"][:Tm] if wait else None, a.pre_ln, cfg.rms_norm_eps,
                      d["resid"][:Tm] if wait else None, d["hs_ptrs"], tp, lo, S.hidden, Tm, S.hidden,
                      wait_flags=d["comb_flag"] if wait else None, n_wait=S.n_expert if wait else 0,
                      wait_epoch=d["comb_epoch"] if wait else None,
                      signal_ptrs=d["hsflag_ptrs"] if tp > 1 else None, n_signal=tp if tp > 1 else 0,
                      signal_slot=self.tp_rank, signal_epoch=d.get("hs_sig_epoch"), ticket=d["ticket"],
                      status=self.status)

    def layer_attn(self, l: int, m: int, parts=("qkv", "attn", "o_proj")) -> None:
        """QKV (+ RoPE + KV append in the epilogue), paged attention, o_proj. With tensor parallelism the QKV GEMM
        consumes the all-gathered rows shard by shard and the o_proj epilogue scatters the partial sums to the rows'
        owners; without it o_proj adds the residual in place. ``parts`` lets a profiler run one of the three launches
        alone (on whatever the buffers hold)."""
        d, S, cfg = self.mb[m], self.shape, self.cfg
        T, per, lo, hi = self.rows(m)
        a = self.layers[l]
        kc, vc = self.kv_cache[l - self.l0, 0], self.kv_cache[l - self.l0, 1]
        meta = self._meta(m)
        rope = gemm.RopeAppend(self.rope, meta.positions, meta.slots, kc, vc, a.num_heads, a.num_kv_heads, a.head_dim)
        if self.tp > 1:
            comm = gemm.GemmComm(shard_rows=per, wait_flags=d["hsflag"], n_wait=self.tp, wait_epoch=d["hs_wait_epoch"],
                                 done_ticket=d["gemm_ticket"], rope=rope)
        else:
            comm = gemm.GemmComm(rope=rope)
        qkv, attn = d["qkv"][:T], d["attn"][:T]
        if "qkv" in parts:
            _lib.TAG = "qkv"
            gemm.linear(d["hs"][:T], a.qkv_w, out=qkv, comm=comm)
            _lib.TAG = ""
        n_pre = self.n_pre[m]
        if "attn" in parts:
            F.paged_attention(qkv[:, :a.q_size], kc, vc, meta.block_tables, meta.bt_row,
                              d["ctx_dec"][:T] if n_pre else meta.ctx_len,
                              a.num_heads, a.num_kv_heads, a.head_dim, out=attn,
                              splits=F.pick_attn_splits(T, a.num_kv_heads, cfg.max_seq_len, self.block_size))
            if n_pre:
                F.prefill_attention(qkv[:, :a.q_size], kc, vc, meta.block_tables, d["pre_tiles"], n_pre, a.num_heads,
                                    a.num_kv_heads, a.head_dim, attn)
        if "o_proj" not in parts:
            return
        _lib.TAG = "o_proj"
        if self.tp == 1:
            gemm.linear(attn, a.o_w, residual=d["resid"][:T], out=d["resid"][:T])
            _lib.TAG = ""
            return
        sig = gemm.GemmComm(rs_bases=d["opart_ptrs"], rs_rows=per, rs_slot=self.tp_rank, rs_cap=S.rows_cap,
                            signal_ptrs=d["oflag_ptrs"], n_signal=self.tp, signal_slot=self.tp_rank,
                            signal_epoch=d["o_sig_epoch"], done_ticket=d["gemm_ticket"])
        gemm.linear(attn, a.o_w, comm=sig)
        _lib.TAG = ""

    def layer_route_dispatch(self, l: int, m: int) -> None:
        """[wait for the TP members' o_proj] reduce + residual, post-attention RMSNorm, router, dispatch of this
        rank's rows: one kernel. Shared experts and dense FFN layers follow on this rank's rows."""
        d, S, cfg = self.mb[m], self.shape, self.cfg
        T, per, lo, hi = self.rows(m)
        Tm = hi - lo
        a = self.layers[l]
        tp = self.tp
        kw = {}
        if tp > 1:
            kw = dict(add=d["opart"], n_add=tp, add_slot_stride=S.rows_cap * S.hidden, ld_add=S.hidden,
                      wait_flags=d["oflag"], n_wait=tp, wait_epoch=d["o_wait_epoch"])
        if not a.is_dense:
            kw.update(x_bases=d["x_bases"], rec_bases=d["rec_bases"], cnt_bases=d["cnt_bases"],
                      flag_bases=d["flag_bases"], ld_dst=S.hidden, experts_per_rank=S.experts_per_rank,
                      n_dst=S.n_expert, my_rank=self.a, region_cap=S.region_cap, disp_epoch=d["disp_epoch"],
                      logit_bias=a.route_bias, topk_ids=d["topk_ids"], topk_w=d["topk_w"])
            if self.stripes > 1:
                # the experts return this layer's output to the stage that owns the next layer (the LM head counts
                # as layer num_layers and belongs to the last stage)
                kw["ret_rank"] = S.layer_owner(l + 1)
        F.route_dispatch(d["resid"], a.post_ln, cfg.rms_norm_eps, None if a.is_dense else a.gate_w, S.top_k,
                         cfg.norm_topk_prob, Tm, y=d["y"], ticket=d["ticket"], status=self.status, **kw)
        if Tm > 0:
            if a.is_dense:
                a.dense_ffn(d["resid"][:Tm], h=d["y"][:Tm])
            else:
                # shared experts stay on the attention GPU and run while the expert GPUs work on the rows just sent
                a.shared_experts(d["y"][:Tm], d["resid"][:Tm])
        if self.stripes > 1 and l == self.l1 - 1 and self.a + 1 < self.stripes:
            self._hand_off(m)

    def _hand_off(self, m: int) -> None:
        """Last layer of this pipeline stage: the residual rows of micro-batch m go to the next stage's residual
        buffer (peer stores) and its hand-off flag is released; the experts send this layer's output there too. One
        launch of the norm + push kernel: the row copy is its residual output, the normalised rows land in a scratch
        buffer nobody reads. Replaces the residual-stream send / recv between pipeline stages of the host-scheduled
        path (the reference's layer striping: disagmoe/utils/placement.py:369-434)."""
        d, S = self.mb[m], self.shape
        T, per, lo, hi = self.rows(m)
        Tm = hi - lo
        F.norm_gather(d["resid"][:Tm], None, self.norm_w, self.cfg.rms_norm_eps, d["ho_next_resid"][:Tm], d["hfin_ptrs"], 1, 0,
                      S.hidden, Tm, S.hidden, signal_ptrs=d["ho_sig_ptrs"], n_signal=1, signal_slot=0,
                      signal_epoch=d["ho_sig_epoch"], ticket=d["ticket"], status=self.status)

    def head(self, m: int) -> None:
        """[wait for the last layer's combine] final norm, LM head and greedy sampling on this rank's rows; a TP group
        then exchanges the sampled ids so that every member holds all of them."""
        d, S, cfg = self.mb[m], self.shape, self.cfg
        if self.stripes > 1 and self.a != self.stripes - 1:
            return      # the last pipeline stage owns the LM head
        T, per, lo, hi = self.rows(m)
        Tm = hi - lo
        wait = self._expert_parts(cfg.num_layers)
        F.norm_gather(d["resid"][:Tm], d["parts"][:Tm] if wait else None, self.norm_w, cfg.rms_norm_eps,
                      d["resid"][:Tm] if wait else None, d["hfin_ptrs"], 1, 0, S.hidden, Tm, S.hidden,
                      wait_flags=d["comb_flag"] if wait else None, n_wait=S.n_expert if wait else 0,
                      wait_epoch=d["comb_epoch"] if wait else None, ticket=d["ticket"], status=self.status)
        if Tm > 0:
            _lib.TAG = "lm_head"
            logits = gemm.linear(d["hfin"][:Tm], self.lm_head_w, out=d["logits"][:Tm], out_dtype=torch.float32)
            _lib.TAG = ""
            F.argmax(logits, out=d["next_local"][:Tm])
        if self.tp > 1:
            F.ids_gather(d["next_local"], Tm, d["nid_ptrs"], self.tp, lo, d["nidflag_ptrs"], self.tp_rank,
                         d["nid_sig_epoch"])

    def head_wait(self, m: int) -> None:
        """A TP group's iteration ends when every member's sampled ids have landed in this rank's id buffer."""
        if self.tp > 1:
            d = self.mb[m]
            F.wait_flags(d["nidflag"], self.tp, d["nid_wait_epoch"], self.status)

    def iteration(self) -> None:
        S = self.shape
        for m in range(S.n_mb):
            self.embed(m)
        for l in range(self.cfg.num_layers):
            for m in range(S.n_mb):
                self.layer(l, m)
        for m in range(S.n_mb):
            self.head(m)
        for m in range(S.n_mb):
            self.head_wait(m)


class ExpertRank:
    """One EP shard of every layer's routed experts."""

    def __init__(self, cfg: ModelConfig, shape: DisaggShape, arena: PeerArena, layout: ArenaLayout, expert_rank: int,
                 state_dict: Optional[W.StateDict] = None, device=None):
        self.cfg, self.shape, self.arena, self.layout, self.x = cfg, shape, arena, layout, expert_rank
        dev = device or arena.local.device
        self.device = dev
        S = shape
        epr = S.experts_per_rank
        self.layers: List[MoEExperts] = []
        for l in range(cfg.num_layers):
            if cfg.is_dense_layer(l):
                self.layers.append(None)
                continue
            e = MoEExperts(cfg, l, expert_rank * epr, min((expert_rank + 1) * epr, cfg.num_experts), device=dev,
                           dtype=torch.bfloat16)
            e.load_weights(state_dict) if state_dict is not None else e.init_weights()
            self.layers.append(e)
        rows = epr * S.region_cap
        z = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        self.act = torch.zeros(rows, cfg.intermediate_size, dtype=torch.bfloat16, device=dev)
        self.ticket = z(1)
        attn_ranks = list(range(S.n_attn))
        self.mb = []
        for m in range(S.n_mb):
            self.mb.append(dict(
                rows=arena.view(layout.offset(f"recv_rows{m}"), (rows, S.hidden), torch.bfloat16),
                recs=arena.view(layout.offset(f"recv_recs{m}"), (rows, 4), torch.int32),
                cnt=arena.view(layout.offset(f"recv_cnt{m}"), (epr,), torch.int32),
                flag=arena.view(layout.offset(f"disp_flag{m}"), (S.n_attn,), torch.int32),
                # one epoch counter per attention rank: with layer striping a layer's rows come from (and go back to) one
                # pipeline stage only, and every stage counts its own hand-shakes; without it slot 0 counts for all
                wait_epoch=z(S.n_attn), signal_epoch=z(S.n_attn),
                parts_bases=arena.ptr_table(attn_ranks, layout.offset(f"parts{m}")),
                signal_ptrs=arena.ptr_table(attn_ranks, layout.offset(f"comb_flag{m}")),
            ))
        pairs = S.n_attn * S.rows_cap * S.top_k              # (token, k) pairs arriving per launch, all experts
        hint = gemm._group_hint(pairs, S.num_experts)
        self.bn = gemm.pick_bn(hint, gemm.EPI_SWIGLU)          # GEMM-1 holds two accumulators per tile: tokens <= 128
        self.bn2 = gemm.pick_bn(hint, gemm.EPI_COMBINE)        # GEMM-2: up to 256 tokens per weight tile
        # work distribution of GEMM-2 from the rows EXPECTED per launch (the receive regions are sized for the worst case)
        n_local = min((expert_rank + 1) * epr, cfg.num_experts) - expert_rank * epr
        self.sk2 = gemm.want_streamk(gemm.EPI_COMBINE, S.hidden, n_local, pairs * n_local // S.num_experts, self.bn2,
                                     gemm.num_sms(dev))

    def layer(self, l: int, m: int) -> None:
        d, S = self.mb[m], self.shape
        e = self.layers[l]
        if e is None:
            return
        if S.stripes > 1:
            # layer striping: only the stage that owns layer l dispatches it, only the owner of layer l + 1 is told
            src, dst = S.layer_owner(l), S.layer_owner(l + 1)
            flags, n_wait, wait_epoch = d["flag"][src:src + 1], 1, d["wait_epoch"][src:src + 1]
            sig_ptrs, n_sig, sig_epoch = d["signal_ptrs"][dst:dst + 1], 1, d["signal_epoch"][dst:dst + 1]
        else:
            flags, n_wait, wait_epoch = d["flag"], S.n_attn, d["wait_epoch"][:1]
            sig_ptrs, n_sig, sig_epoch = d["signal_ptrs"], S.n_attn, d["signal_epoch"][:1]
        gate = gemm.GemmComm(seg_cnt=d["cnt"], seg_cap=S.region_cap, group_regions=True, wait_flags=flags,
                             n_wait=n_wait, wait_epoch=wait_epoch, done_ticket=self.ticket)
        _lib.TAG = "expert_gemm1"
        gemm.grouped_swiglu(d["rows"], e.w13_weight, None, out=self.act, bn=self.bn, comm=gate, w_blocked=e.w_blocked)
        _lib.TAG = "expert_gemm2"
        # the last CTA clears the row cursors before it signals: the senders reserve again only after that signal
        sig = gemm.GemmComm(seg_cnt=d["cnt"], seg_cap=S.region_cap, group_regions=True, signal_ptrs=sig_ptrs,
                            n_signal=n_sig, signal_slot=self.x, signal_epoch=sig_epoch,
                            done_ticket=self.ticket, clear=d["cnt"])
        gemm.grouped_combine(self.act, e.w2_weight, None, d["recs"], d["parts_bases"], S.hidden, bn=self.bn2, comm=sig,
                             streamk=self.sk2, w_blocked=e.w_blocked)
        _lib.TAG = ""

    def iteration(self) -> None:
        for l in range(self.cfg.num_layers):
            for m in range(self.shape.n_mb):
                self.layer(l, m)


def selfcheck_against_colocated(world: int, rank: int, local_rank: int, n_attn: int, tp: int, n_mb: int = 2,
                                batch: int = 8, stripes: int = 1) -> Dict[str, float]:
    """Correctness line of a multi-GPU job: a tiny model (2 layers, hidden 256, 8 experts) runs one decode iteration
    through the fused pipeline on the job's real GPUs with the job's layout (attention groups, TP degree, expert
    GPUs), and every attention rank compares the logits of the rows it owns with the single-GPU colocated executor
    fed the same weights, KV history and inputs. Collective over the world; returns the worst relative error
    (max |diff| / max |ref|) and the worst fraction of rows whose arg-max agrees, over all ranks. With ``stripes`` =
    n_attn the attention GPUs run as one pipeline over 2 x stripes layers and the last stage holds the logits."""
    import torch.distributed as dist
    from ..config import CacheConfig, tiny_config
    from ..executor.fused import FusedModelExecutor
    A, X = n_attn, world - n_attn
    cfg = tiny_config.clone(dtype=torch.bfloat16, num_layers=2 if stripes <= 1 else 2 * stripes)
    dev = torch.device("cuda", local_rank)
    sd = {k: v.to(torch.bfloat16) for k, v in W.init_state_dict(cfg, dtype=torch.float32).items()}
    B = batch * tp
    shape = DisaggShape(A, X, n_mb, B, cfg.top_k, cfg.hidden_size, cfg.num_experts, tp, stripes=stripes,
                        num_layers=cfg.num_layers)
    layout = build_layout(shape)
    arena = PeerArena.create(layout.size, device=dev)
    nb, bs = 4 * n_mb * B + 1, 16
    err, agree, err_close, rows_close, rows_total = 0.0, 1.0, 0.0, 0, 0
    if rank < A:
        grp = rank // tp if stripes <= 1 else 0      # the stages of a pipeline serve the same requests
        g = torch.Generator().manual_seed(99 + grp)
        r = AttentionRank(cfg, shape, arena, layout, rank, nb, state_dict=sd, device=dev)
        kvh = cfg.num_kv_heads // tp if cfg.num_kv_heads >= tp else 1
        kv = torch.randn(cfg.num_layers, 2, nb, bs, cfg.num_kv_heads, cfg.head_dim, generator=g).to(torch.bfloat16) * 0.5
        k0 = (rank % tp) * kvh if cfg.num_kv_heads >= tp else (rank % tp) // (tp // cfg.num_kv_heads)
        r.kv_cache.copy_(kv[r.l0:r.l1, ..., k0:k0 + kvh, :])
        inputs = []
        for m in range(n_mb):
            ids = torch.randint(0, cfg.vocab_size, (B,), generator=g).int()
            ctx = torch.randint(3, 60, (B,), generator=g).int()
            bt = (torch.arange(B * 4, dtype=torch.int32) + m * B * 4).view(B, 4)
            slots = torch.tensor([int(bt[i, int(ctx[i]) // bs]) * bs + int(ctx[i]) % bs for i in range(B)])
            rows = torch.arange(B, dtype=torch.int32) + m * B
            r.block_tables[m * B:(m + 1) * B, :4] = bt.to(dev)
            d = r.mb[m]
            d["ids"].copy_(ids); d["positions"].copy_(ctx); d["ctx_len"].copy_(ctx + 1)
            d["bt_row"].copy_(rows); d["slots"].copy_(slots)
            inputs.append((ids, ctx, slots, bt))
    else:
        r = ExpertRank(cfg, shape, arena, layout, rank - A, state_dict=sd, device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    r.iteration()
    torch.cuda.synchronize()
    dist.barrier()
    status = gemm.check_status(dev)
    if rank < A:
        ref = FusedModelExecutor(cfg, CacheConfig(block_size=bs), device=dev, max_batch_size=B, max_prefill_tokens=B,
                                 state_dict=sd, num_blocks=nb, enable_cuda_graph=False)
        per = shard_rows(B, tp)
        lo, hi = min(B, (rank % tp) * per), min(B, (rank % tp + 1) * per)
        if stripes > 1 and rank != A - 1:
            inputs = []                             # only the last stage of a pipeline holds logits
        for m, (ids, ctx, slots, bt) in enumerate(inputs):
            ref.kv_cache.copy_(kv)
            ref.block_tables[:B, :4] = bt.to(dev)
            _, lg = ref.decode(ids, ctx, slots, ctx + 1, torch.arange(B, dtype=torch.int32), want_logits=True)
            got, want = r.mb[m]["logits"][:hi - lo].float(), lg[lo:hi].float()
            if hi > lo:
                row_err = (got - want).abs().amax(-1) / want.abs().max()
                err = max(err, float(row_err.max()))
                agree = min(agree, float((got.argmax(-1) == want.argmax(-1)).float().mean()))
                rows_total += hi - lo
                close = row_err < 0.02
                rows_close += int(close.sum())
                if bool(close.any()):
                    err_close = max(err_close, float(row_err[close].max()))
        torch.cuda.synchronize()
    t = torch.tensor([err, -agree, float(status), err_close], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    n = torch.tensor([rows_close, rows_total], device=dev, dtype=torch.float64)
    dist.all_reduce(n)
    return {"max_rel_err": round(float(t[0]), 5), "argmax_agree_min": round(-float(t[1]), 4), "kernel_status": int(t[2]),
            "rows_within_2pct": int(n[0]), "rows": int(n[1]), "max_rel_err_of_those_rows": round(float(t[3]), 5),
            "model": f"tiny {cfg.num_layers}-layer MoE, same GPU layout, vs the colocated executor; a row outside 2 % is a router near-tie "
                     "that flips under the TP group's bf16 summation order (benchmark/emulated_selfcheck.py runs the same "
                     "layout sequentially on one GPU for comparison)"}


class DisaggDecodeBench:
    """Decode-throughput runner used by ``bench.py`` for N >= 2 GPUs (one process per GPU, NCCL only for bootstrap)."""

    def __init__(self, cfg: ModelConfig, world: int, rank: int, local_rank: int, batch: int, ctx_min: int, ctx_max: int,
                 total_steps: int, gen: torch.Generator, n_mb: int = 2, tp: int = 1, n_attn: int = 0,
                 route_skew: float = 0.0):
        import torch.distributed as dist
        A = n_attn or world // 2
        X = world - A
        assert 1 <= A < world and A % tp == 0, "ranks [0, A) are attention GPUs, the rest hold experts"
        assert (X - 1) * ((cfg.num_experts + X - 1) // X) < cfg.num_experts, "an expert GPU would hold no expert"
        self.cfg, self.world, self.rank = cfg, world, rank
        # a TP group of `tp` attention GPUs serves tp x batch sequences per micro-batch (per-GPU load stays `batch`)
        batch = batch * tp
        self.shape = DisaggShape(A, X, n_mb, batch, cfg.top_k, cfg.hidden_size, cfg.num_experts, tp)
        self.tp = tp
        if tp > 1 and rank < A:
            gen = torch.Generator().manual_seed(4321 + rank // tp)    # every member of a TP group sees the same requests
        self.layout = build_layout(self.shape)
        self.device = torch.device("cuda", local_rank)
        self.arena = PeerArena.create(self.layout.size, device=self.device)
        self.is_attn = rank < A
        self.parallelism = f"attn dp{A // tp}" + (f" x tp{tp}" if tp > 1 else "") + \
            f" x {n_mb} micro-batches + expert ep{X} (up to {self.shape.experts_per_rank} experts/GPU), " \
            "fused peer-memory dispatch/combine" + (f", Zipf({route_skew}) expert popularity" if route_skew > 0 else "")
        self.h2d_bytes_last = self.d2h_bytes_last = 0
        self.profile_events = False
        self.event_pairs = []
        self._launch0 = 0
        B = batch
        if self.is_attn:
            ctx = torch.randint(ctx_min, ctx_max + 1, (n_mb * B,), generator=gen).tolist()
            blocks = sum((c + total_steps + 2 + 15) // 16 for c in ctx) + 64
            self.runner = AttentionRank(cfg, self.shape, self.arena, self.layout, rank, blocks)
            for layer in self.runner.layers:
                layer.set_route_skew(route_skew)
            self.runner.kv_cache.normal_(0, 0.5)
            self.block_mgr = C.BlockManager(16, blocks, 0, n_mb * B)
            self.lens = ctx
            self.last = torch.randint(0, cfg.vocab_size, (n_mb * B,), generator=gen).tolist()
            for i in range(n_mb * B):
                self.block_mgr.allocate(i, ctx[i] + 1)
            n = n_mb * B
            pin = lambda dt: torch.zeros(n, dtype=dt, pin_memory=True)
            self.h_ids, self.h_pos, self.h_ctx, self.h_row, self.h_slots = pin(torch.int32), pin(torch.int32), \
                pin(torch.int32), pin(torch.int32), pin(torch.int64)
            self.h_out = pin(torch.int32)
            self._patch_tables()
        else:
            self.runner = ExpertRank(cfg, self.shape, self.arena, self.layout, rank - A)
        torch.cuda.synchronize()
        dist.barrier()
        # eager warm-up in lock step (sizes scratch buffers, sets kernel attributes), then capture
        for _ in range(2):
            if self.is_attn:
                self._stage_inputs(advance=False)
            self.runner.iteration()
            torch.cuda.synchronize()
            dist.barrier()
        self.graph = torch.cuda.CUDAGraph()
        n0 = _lib.LAUNCHES
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.graph(self.graph, stream=side):
            self.runner.iteration()
        self.graph_launches = _lib.LAUNCHES - n0
        torch.cuda.synchronize()
        dist.barrier()

    # ---- host side of an attention rank ------------------------------------------------------------------------
    def _patch_tables(self) -> int:
        ups = self.block_mgr.drain_updates()
        if not ups:
            return 0
        t = torch.tensor(ups, dtype=torch.int64).T.contiguous().pin_memory().to(self.device, non_blocking=True)
        self.runner.block_tables.index_put_((t[0], t[1]), t[2].int())
        return 24 * len(ups)

    def _stage_inputs(self, advance: bool) -> int:
        n = len(self.lens)
        B = self.shape.batch
        rs = self.block_mgr.step_decode(list(range(n)), self.lens)
        self.h_ids.numpy()[:] = self.last
        self.h_pos.numpy()[:] = self.lens
        self.h_ctx.numpy()[:] = [l + 1 for l in self.lens]
        self.h_row.numpy()[:] = rs[:n]
        self.h_slots.numpy()[:] = rs[n:]
        nbytes = self._patch_tables()
        for m, d in enumerate(self.runner.mb):
            sl = slice(m * B, (m + 1) * B)
            d["ids"].copy_(self.h_ids[sl], non_blocking=True)
            d["positions"].copy_(self.h_pos[sl], non_blocking=True)
            d["ctx_len"].copy_(self.h_ctx[sl], non_blocking=True)
            d["bt_row"].copy_(self.h_row[sl], non_blocking=True)
            d["slots"].copy_(self.h_slots[sl], non_blocking=True)
        return nbytes + n * 24

    def step(self) -> None:
        ev = None
        if self.profile_events:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        self.h2d_bytes_last = self.d2h_bytes_last = 0
        if self.is_attn:
            B = self.shape.batch
            if ev:
                ev[0].record()
            self.h2d_bytes_last = self._stage_inputs(advance=True)
            self.graph.replay()
            _lib.add_launches(self.graph_launches)
            for m, d in enumerate(self.runner.mb):
                self.h_out[m * B:(m + 1) * B].copy_(d["next_ids"], non_blocking=True)
            if ev:
                ev[1].record()
            torch.cuda.current_stream().synchronize()
            self.last = self.h_out.tolist()
            self.lens = [l + 1 for l in self.lens]
            self.d2h_bytes_last = 4 * len(self.lens)
        else:
            if ev:
                ev[0].record()
            self.graph.replay()
            _lib.add_launches(self.graph_launches)
            if ev:
                ev[1].record()
            torch.cuda.current_stream().synchronize()
        if ev:
            self.event_pairs.append(ev)

    def timeline(self, iterations: int = 2) -> Dict[str, tuple]:
        """Per-kernel device time of ``iterations`` EAGER (not graph-replayed) coupled iterations of this rank, every
        rank of the job taking part: {label: (launches, total ms)}. A kernel's time includes the wait on its peers'
        flags inside it, so the labels show where this rank's pipeline stalls."""
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        _lib.start_timeline()
        for _ in range(iterations):
            if self.is_attn:
                self._stage_inputs(advance=True)
                self.lens = [l + 1 for l in self.lens]
            self.runner.iteration()
        return _lib.stop_timeline()

    def tokens_per_step(self) -> int:
        # a sequence served by a TP group is counted once (by the group's first rank)
        if not self.is_attn or self.rank % self.tp != 0:
            return 0
        return self.shape.n_mb * self.shape.batch

    def launch_count(self) -> int:
        return _lib.LAUNCHES

    def status(self) -> int:
        return gemm.check_status(self.device)
