"""Device-driven disaggregated decode: attention GPUs and expert GPUs exchange tokens through peer memory.

Ranks [0, A) are attention replicas (data parallel, each with its own sequences and KV cache); ranks [A, A + X) hold
the routed experts (expert parallel, ``num_experts / X`` experts each). One decode iteration of a micro-batch is,
per layer:

    attention rank   [wait combine flags]  add+RMSNorm -> QKV -> RoPE/KV append -> paged attention -> o_proj+residual
                     -> RMSNorm+gate+top-k -> dispatch: a block of rows per expert is reserved on the owning expert GPU
                     (one system-scope atomic per expert), then rows, records and a release flag are stored there
    expert rank      grouped GEMM-1 (+SwiGLU), gated on the arrival flags, reads the rows where they landed
                     -> grouped GEMM-2 whose epilogue scales by the router weight and stores every row into the
                     source attention GPU's partial-output buffer, then signals that GPU

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
    batch: int          # sequences per micro-batch
    top_k: int
    hidden: int
    num_experts: int
    tp: int = 1         # attention tensor-parallel degree: consecutive groups of `tp` attention ranks share sequences

    @property
    def experts_per_rank(self) -> int:
        # experts are dealt out in contiguous blocks of ceil(E / X); the last expert rank may hold fewer
        return (self.num_experts + self.n_expert - 1) // self.n_expert

    @property
    def region_cap(self) -> int:   # rows of one expert's receive region: every sender could route all its pairs to it
        return self.n_attn * (self.batch // self.tp) * self.top_k


def build_layout(s: DisaggShape) -> ArenaLayout:
    L = ArenaLayout()
    rows = s.experts_per_rank * s.region_cap
    for m in range(s.n_mb):
        L.add(f"recv_rows{m}", rows * s.hidden * 2)
        L.add(f"recv_recs{m}", rows * 16)
        L.add(f"recv_cnt{m}", s.experts_per_rank * 4)      # per-expert row cursors, advanced by the senders
        L.add(f"disp_flag{m}", s.n_attn * 4)
        L.add(f"parts{m}", s.batch * s.top_k * s.hidden * 2)
        L.add(f"comb_flag{m}", s.n_expert * 4)
        if s.tp > 1:
            # this rank's o_proj partial sums, read by its TP peers. Two buffers used by layer parity: a peer may
            # still read layer l's partials while this rank already writes layer l + 1's (nothing else orders the two
            # when layer l has a dense FFN and so no round trip through the expert GPUs); by layer l + 2 the peer's
            # own layer l + 1 signal proves it is done with layer l
            L.add(f"opart{m}_0", s.batch * s.hidden * 2)
            L.add(f"opart{m}_1", s.batch * s.hidden * 2)
            L.add(f"oflag{m}", s.tp * 4)
    return L


class AttentionRank:
    """All attention layers + embedding + LM head of one DP replica, with its KV cache and micro-batch buffers."""

    def __init__(self, cfg: ModelConfig, shape: DisaggShape, arena: PeerArena, layout: ArenaLayout, attn_rank: int,
                 num_blocks: int, block_size: int = 16, state_dict: Optional[W.StateDict] = None, device=None):
        self.cfg, self.shape, self.arena, self.layout, self.a = cfg, shape, arena, layout, attn_rank
        dev = device or arena.local.device
        self.device = dev
        dt = torch.bfloat16
        self.tp = shape.tp
        self.tp_rank = attn_rank % shape.tp
        self.group0 = attn_rank // shape.tp * shape.tp      # first attention rank of this TP group
        assert shape.batch % shape.tp == 0
        self.layers: List[MoEAttention] = []
        for l in range(cfg.num_layers):
            m = MoEAttention(cfg, l, tp_size=self.tp, tp_rank=self.tp_rank, device=dev, dtype=dt)
            m.load_weights(state_dict) if state_dict is not None else m.init_weights()
            self.layers.append(m)
        names = ["embed_tokens.weight", "norm.weight", "lm_head.weight"]
        sd = state_dict if state_dict is not None else W.init_state_dict(cfg, dev, dt, names)
        self.embed_w = sd["embed_tokens.weight"].to(device=dev, dtype=dt).contiguous()
        self.norm_w = sd["norm.weight"].to(device=dev, dtype=dt)
        self.lm_head_w = sd["lm_head.weight"].to(device=dev, dtype=dt).contiguous()
        S = shape
        B, k, H, E = S.batch, S.top_k, S.hidden, S.num_experts
        self.block_size = block_size
        self.max_blocks = (cfg.max_seq_len + block_size - 1) // block_size
        self.kv_cache = torch.zeros(cfg.num_layers, 2, num_blocks, block_size, self.layers[0].num_kv_heads, cfg.head_dim,
                                    dtype=dt, device=dev)
        self.block_tables = torch.zeros(S.n_mb * B, self.max_blocks, dtype=torch.int32, device=dev)
        z = lambda *s, dt_=torch.int32: torch.zeros(*s, dtype=dt_, device=dev)
        self.mb = []
        expert_ranks = [S.n_attn + x for x in range(S.n_expert)]
        for m in range(S.n_mb):
            d = dict(
                ids=z(B), positions=z(B), slots=z(B, dt_=torch.int64), ctx_len=z(B), bt_row=z(B),
                resid=torch.zeros(B, H, dtype=dt, device=dev), ws=z(3 * E + 8), disp_epoch=z(1), wait_epoch=z(1),
                next_ids=z(B), logits=torch.zeros(B, cfg.vocab_size, dtype=torch.float32, device=dev),
                parts=arena.view(layout.offset(f"parts{m}"), (B, k, H), dt),
                comb_flag=arena.view(layout.offset(f"comb_flag{m}"), (S.n_expert,), torch.int32),
                x_bases=arena.ptr_table(expert_ranks, layout.offset(f"recv_rows{m}")),
                rec_bases=arena.ptr_table(expert_ranks, layout.offset(f"recv_recs{m}")),
                cnt_bases=arena.ptr_table(expert_ranks, layout.offset(f"recv_cnt{m}")),
                flag_bases=arena.ptr_table(expert_ranks, layout.offset(f"disp_flag{m}")),
            )
            if self.tp > 1:
                group = [self.group0 + i for i in range(self.tp)]
                d.update(
                    opart=[arena.view(layout.offset(f"opart{m}_{p}"), (B, H), dt) for p in range(2)],
                    oflag=arena.view(layout.offset(f"oflag{m}"), (self.tp,), torch.int32),
                    opart_ptrs=[arena.ptr_table(group, layout.offset(f"opart{m}_{p}")) for p in range(2)],
                    oflag_ptrs=arena.ptr_table(group, layout.offset(f"oflag{m}")),
                    o_signal_epoch=z(1), o_wait_epoch=z(1), o_ticket=z(1),
                    y=torch.zeros(B, H, dtype=dt, device=dev), topk_ids=z(B, k),
                    topk_w=torch.zeros(B, k, dtype=torch.float32, device=dev))
            self.mb.append(d)
        self.status = gemm.scratch(dev).status
        self.active = [B] * S.n_mb      # rows of every micro-batch that the next launches process (<= B)
        self._views: Dict[tuple, dict] = {}

    _ROW_KEYS = ("ids", "positions", "slots", "ctx_len", "bt_row", "resid", "next_ids", "logits", "parts", "y",
                 "topk_ids", "topk_w")

    def set_active(self, m: int, T: int) -> None:
        """The next launches of micro-batch m process its first T rows (1 <= T <= batch): a serving step fills the
        buffers with however many decode and prompt tokens it scheduled."""
        assert 1 <= T <= self.shape.batch
        self.active[m] = T

    def _d(self, m: int) -> dict:
        T = self.active[m]
        full = self.mb[m]
        if T == self.shape.batch:
            return full
        v = self._views.get((m, T))
        if v is None:
            v = dict(full)
            for k in self._ROW_KEYS:
                if k in full:
                    v[k] = full[k][:T]
            if "opart" in full:
                v["opart"] = [t[:T] for t in full["opart"]]
            self._views[(m, T)] = v
        return v

    def _meta(self, m: int) -> AttnMeta:
        d = self._d(m)
        return AttnMeta(d["positions"], d["slots"], self.block_tables, d["bt_row"], d["ctx_len"],
                        max_ctx=self.cfg.max_seq_len)

    def embed(self, m: int) -> None:
        d = self._d(m)
        F.embed(d["ids"], self.embed_w, out=d["resid"])

    def layer(self, l: int, m: int) -> None:
        """Attention half of layer l for micro-batch m, ending with the peer-memory dispatch."""
        self.layer_attn(l, m)
        self.layer_route_dispatch(l, m)

    def layer_attn(self, l: int, m: int) -> None:
        """[wait for the experts' combine] add + RMSNorm, QKV, RoPE / KV append, paged attention, o_proj. With tensor
        parallelism the o_proj partial sum goes to this rank's peer-visible buffer and the GEMM signals the TP peers."""
        d, S, cfg = self._d(m), self.shape, self.cfg
        T = self.active[m]
        parts = None
        if l > 0 and not cfg.is_dense_layer(l - 1):     # a dense-FFN layer sends nothing to the expert GPUs
            _lib.check(_lib.lib().dmoe_wait_flags(_vp(d["comb_flag"]), c_int(S.n_expert), _vp(d["wait_epoch"]),
                                                  _vp(self.status), c_vp(_lib.stream_ptr())), "dmoe_wait_flags")
            parts = d["parts"]
        a = self.layers[l]
        kv = (self.kv_cache[l, 0], self.kv_cache[l, 1])
        if self.tp == 1:
            d["resid2"] = a.attention(d["resid"], parts, kv, self._meta(m))
            return
        meta = self._meta(m)
        resid, h = F.add_rmsnorm(d["resid"], parts, a.pre_ln, cfg.rms_norm_eps, resid_out=d["resid"])
        qkv = gemm.linear(h, a.qkv_w)
        F.rope_kv_append(qkv, meta.positions, meta.slots, kv[0], kv[1], a.num_heads, a.num_kv_heads, a.head_dim,
                         cfg.rope_theta)
        attn = F.paged_attention(qkv[:, :a.q_size], kv[0], kv[1], meta.block_tables, meta.bt_row, meta.ctx_len,
                                 a.num_heads, a.num_kv_heads, a.head_dim,
                                 splits=F.pick_attn_splits(T, a.num_kv_heads, cfg.max_seq_len, self.block_size))
        sig = gemm.GemmComm(signal_ptrs=d["oflag_ptrs"], n_signal=self.tp, signal_slot=self.tp_rank,
                            signal_epoch=d["o_signal_epoch"], done_ticket=d["o_ticket"])
        gemm.linear(attn, a.o_w, out=d["opart"][l % 2], comm=sig)

    def layer_route_dispatch(self, l: int, m: int) -> None:
        """Post-attention RMSNorm + router + dispatch. With tensor parallelism the router kernel first sums the TP
        ranks' o_proj partials straight out of their memory (the all-reduce), and this rank dispatches only its
        slice of the tokens."""
        d, S, cfg = self._d(m), self.shape, self.cfg
        T = self.active[m]
        a = self.layers[l]
        lo, hi = 0, T
        if a.is_dense and self.tp == 1:
            a.dense_ffn(d["resid"])
            return
        if self.tp == 1:
            a.counts = d["ws"][:S.num_experts]
            y, ids, w, _ = a.route(d["resid2"])
        else:
            _lib.check(_lib.lib().dmoe_wait_flags(_vp(d["oflag"]), c_int(self.tp), _vp(d["o_wait_epoch"]),
                                                  _vp(self.status), c_vp(_lib.stream_ptr())), "dmoe_wait_flags")
            per = (T + self.tp - 1) // self.tp
            lo, hi = min(T, self.tp_rank * per), min(T, (self.tp_rank + 1) * per)
            y, ids, w = d["y"], d["topk_ids"], d["topk_w"]
            _lib.check(_lib.lib().dmoe_route_ex(
                _vp(d["resid"]), c_ll(S.hidden), _vp(a.post_ln), ctypes.c_float(cfg.rms_norm_eps), _vp(a.gate_w),
                c_int(T), c_int(S.hidden), c_int(S.num_experts), c_int(S.top_k), c_int(int(cfg.norm_topk_prob)),
                _vp(y), c_ll(S.hidden), _vp(ids), _vp(w), _vp(d["ws"]), _vp(d["opart_ptrs"][l % 2]), c_int(self.tp),
                c_ll(S.hidden), _vp(d["resid"]), c_ll(S.hidden), c_int(lo), c_int(hi), _vp(a.route_bias),
                c_vp(_lib.stream_ptr())), "dmoe_route_ex")
            if a.is_dense:
                # the router kernel ran without a gate: it summed the TP partials into the residual stream and
                # normalised it; every TP rank then applies the (replicated) dense FFN to all rows
                a.dense_ffn(d["resid"], h=y)
                return
        _lib.check(_lib.lib().dmoe_dispatch_remote(
            _vp(y), c_ll(y.stride(0)), _vp(ids), _vp(w), c_int(T), c_int(S.top_k), c_int(S.hidden),
            c_int(S.num_experts), c_int(S.experts_per_rank), c_int(S.n_expert), c_int(self.a), c_int(S.region_cap),
            _vp(d["ws"]), _vp(d["x_bases"]), c_ll(S.hidden), _vp(d["rec_bases"]), _vp(d["cnt_bases"]),
            _vp(d["flag_bases"]), _vp(d["disp_epoch"]), _vp(self.status), c_int(lo), c_int(hi),
            c_vp(_lib.stream_ptr())), "dmoe_dispatch_remote")
        # shared experts stay on the attention GPU and run while the expert GPUs work on the rows just sent
        # (replicated over the ranks of a TP group)
        a.shared_experts(y, d["resid"])

    def head(self, m: int) -> None:
        d, S, cfg = self._d(m), self.shape, self.cfg
        _lib.check(_lib.lib().dmoe_wait_flags(_vp(d["comb_flag"]), c_int(S.n_expert), _vp(d["wait_epoch"]),
                                              _vp(self.status), c_vp(_lib.stream_ptr())), "dmoe_wait_flags")
        _, h = F.add_rmsnorm(d["resid"], d["parts"], self.norm_w, cfg.rms_norm_eps, resid_out=d["resid"])
        logits = gemm.linear(h, self.lm_head_w, out=d["logits"], out_dtype=torch.float32)
        F.argmax(logits, out=d["next_ids"])

    def iteration(self) -> None:
        S = self.shape
        for m in range(S.n_mb):
            self.embed(m)
        for l in range(self.cfg.num_layers):
            for m in range(S.n_mb):
                self.layer(l, m)
        for m in range(S.n_mb):
            self.head(m)


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
                wait_epoch=z(1), signal_epoch=z(1),
                parts_bases=arena.ptr_table(attn_ranks, layout.offset(f"parts{m}")),
                signal_ptrs=arena.ptr_table(attn_ranks, layout.offset(f"comb_flag{m}")),
            ))
        pairs = S.n_attn * (S.batch // S.tp) * S.top_k       # (token, k) pairs arriving per launch, all experts
        self.bn = gemm.pick_bn(gemm._group_hint(pairs, S.num_experts), gemm.EPI_SWIGLU)

    def layer(self, l: int, m: int) -> None:
        d, S = self.mb[m], self.shape
        e = self.layers[l]
        if e is None:
            return
        gate = gemm.GemmComm(seg_cnt=d["cnt"], seg_cap=S.region_cap, group_regions=True, wait_flags=d["flag"],
                             n_wait=S.n_attn, wait_epoch=d["wait_epoch"], done_ticket=self.ticket)
        gemm.grouped_swiglu(d["rows"], e.w13_weight, None, out=self.act, bn=self.bn, comm=gate)
        # the last CTA clears the row cursors before it signals: the senders reserve again only after that signal
        sig = gemm.GemmComm(seg_cnt=d["cnt"], seg_cap=S.region_cap, group_regions=True, signal_ptrs=d["signal_ptrs"],
                            n_signal=S.n_attn, signal_slot=self.x, signal_epoch=d["signal_epoch"],
                            done_ticket=self.ticket, fanout=S.tp, clear=d["cnt"])
        gemm.grouped_combine(self.act, e.w2_weight, None, d["recs"], d["parts_bases"], S.hidden, bn=self.bn, comm=sig)

    def iteration(self) -> None:
        for l in range(self.cfg.num_layers):
            for m in range(self.shape.n_mb):
                self.layer(l, m)


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

    def tokens_per_step(self) -> int:
        # a sequence served by a TP group is counted once (by the group's first rank)
        if not self.is_attn or self.rank % self.tp != 0:
            return 0
        return self.shape.n_mb * self.shape.batch

    def launch_count(self) -> int:
        return _lib.LAUNCHES

    def status(self) -> int:
        return gemm.check_status(self.device)
