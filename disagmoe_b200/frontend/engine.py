"""Per-device worker: the host-scheduled, layer-by-layer engine of the disaggregated deployment.

Every worker owns the native runtime of its role(s) -- receive pool, layer scheduler, dispatcher
(:mod:`disagmoe_b200.disagmoe_c`) -- and a Python loop that asks the scheduler for the next layer's batch, runs the
layer's module and hands the result to the dispatcher. Tokens flow asynchronously: there is no global step.

    attention worker   batch = complete tokens of one layer (their partial rows: top-k expert outputs + the residual
                       part). Sum + RMSNorm, attention, o_proj, router; the k routed copies go to the expert workers
                       (sorted by expert), the residual stream goes to the attention worker of the next layer.
                       Layer ``num_layers`` is the LM-head step: final norm, logits, greedy token -> sampler.
    expert worker      batch = rows of one layer sorted by local expert; grouped SwiGLU FFN, router-weight scale,
                       rows returned to the attention replica (dp rank) that owns each sequence.

Counterpart of disagmoe/frontend/engine.py:47-1089 (Engine, SamplerEngine, TokenizerEngine). What is different on
purpose: real model semantics (embedding, positions, prefill over all prompt tokens, residual stream, LM head), no
busy-spinning on the scheduler (the loop blocks in a GIL-free native wait), clean shutdown, any device (CPU fp32 for
the correctness configuration, CUDA bf16 with the sm_100a kernels).
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .. import disagmoe_c as C
from ..config import CacheConfig, ModelConfig
from ..models import weights as W
from ..models.attention import AttnMeta, MoEAttention
from ..models.experts import MoEExperts, MoEExpertsSerial
from ..ops import functional as F
from ..ops import gemm
from .datatypes import SloStat
from ..utils.logger import get_logger
from ..utils.metrics import Metric
from ..utils.placement import ModelPlacement
from ..utils.utils import StepInfo, Timer, nvtx_range, time_ms


@dataclass
class InitCoreArgs:
    """Everything a worker needs to build its native runtime (the role of the argument list of
    ``Engine.init_core`` at disagmoe/frontend/engine.py:180-269)."""
    layer_ids: List[int]
    in_device_ids: List[int]
    out_device_ids: List[int]
    out_channel_infos: List[Tuple[List[Tuple[int, int]], List[int], int]]
    in_nccl_ids: Dict[int, bytes] = field(default_factory=dict)
    out_nccl_ids: Dict[int, bytes] = field(default_factory=dict)
    attn_peer: Dict[int, Dict[int, int]] = field(default_factory=dict)     # layer -> dp rank -> device
    expert_ranks: List[Tuple[int, int, int]] = field(default_factory=list)
    local_attn_dp_rank: int = 0
    expert_ids: List[Tuple[int, int]] = field(default_factory=list)       # (layer, expert) run here
    hosts: Dict[int, str] = field(default_factory=dict)
    port_shift: int = 0
    state_dict_path: Optional[str] = None
    keep_logits: bool = False
    # attention tensor parallelism of the host-scheduled path: rank 0 of a group (the driver) takes part in the token
    # flow and broadcasts every attention batch it schedules to the other ranks (the workers) of its group
    tp_rank: int = 0
    tp_size: int = 1
    tp_master_port: int = 0


class _EngineLayers:
    """The engine's attention layers and KV caches behind the executor interface that ``CUDAGraphAttnExecutor`` drives."""

    def __init__(self, engine: "Engine", layer_ids):
        self.engine, self.layer_ids = engine, list(layer_ids)
        self.device, self.dtype = engine.device, engine.dtype

    def execute(self, layer_id, positions, hidden_states, meta, parts=None):
        e = self.engine
        meta.positions = positions
        out = e.attn_layers[layer_id].forward(hidden_states, parts, (e.kv_cache[layer_id][0], e.kv_cache[layer_id][1]), meta)
        return out.expert_input, out.topk_weights, out.topk_ids


class Engine:
    def __init__(self, device_id: int = 0, device: str = "cpu"):
        self.device_id = device_id
        self.device = torch.device(device)
        self.model_config: Optional[ModelConfig] = None
        self.cache_config: Optional[CacheConfig] = None
        self.handles = None
        self.attn_layers: Dict[int, MoEAttention] = {}
        self.expert_layers: Dict[int, MoEExperts] = {}
        self.block_mgr = None
        self.kv_cache = None
        self.loop_thread: Optional[threading.Thread] = None
        self.end_flag = False
        self.metric = Metric()
        self.step_infos: List[StepInfo] = []
        self.timer = Timer()
        self.logits_log: Dict[Tuple[int, int], torch.Tensor] = {}
        self._logger = get_logger(f"engine{device_id}")
        self.error: Optional[str] = None
        self._max_rows = 1024
        self.tp_rank, self.tp_size = 0, 1
        self._queueing_delays: List[float] = []      # per executed step: how long its oldest row waited (ms)
        self.has_attn = self.has_expert = False

    # ---- set-up ---------------------------------------------------------------------------------------------
    def set_hosts(self, pid_tag: int, hosts: Dict[int, str]) -> None:
        C.set_hosts(pid_tag, hosts)

    def setup_engine(self, model_config: ModelConfig, cache_config: CacheConfig, dtype: Optional[torch.dtype] = None,
                     inproc: bool = False) -> None:
        self.model_config, self.cache_config = model_config, cache_config
        self.dtype = dtype or model_config.dtype
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        C.set_inproc_transport(inproc)

    def init_core(self, args: InitCoreArgs, placement: ModelPlacement) -> None:
        cfg = self.model_config
        L = cfg.num_layers
        C.set_port_base(args.port_shift)
        if args.hosts:
            C.set_hosts(os.getpid(), args.hosts)
        self.args = args
        self.tp_rank, self.tp_size = args.tp_rank, args.tp_size
        if self.tp_size > 1:
            self._init_tp_group(args)
        self.has_attn = placement.has_attn(self.device_id)
        self.has_expert = placement.has_expert(self.device_id)
        self.dp_rank = args.local_attn_dp_rank
        ea = C.EngineArgs()
        ea.local_id, ea.top_k = self.device_id, cfg.top_k
        ea.has_attn, ea.has_expert = self.has_attn, self.has_expert
        pc = C.ParallelConfig()
        pc.tp, pc.ep, pc.dp, pc.n_exp_per_rank = cfg.tp_size, cfg.ep_size, cfg.dp_size, cfg.num_experts_per_rank
        pc.expert_ranks = [tuple(t) for t in args.expert_ranks]
        ea.cfg = pc
        attn_layers = sorted(placement.attn_layer_ids_at(self.device_id)) if self.has_attn else []
        self.hosts_head = self.has_attn and args.attn_peer.get(L, {}).get(self.dp_rank) == self.device_id
        ea.attn_layer_ids = attn_layers + ([L] if self.hosts_head else [])
        self.local_experts: Dict[int, List[int]] = {}
        for l, e in args.expert_ids:
            self.local_experts.setdefault(l, []).append(e)
        ea.expert_layer_ids = sorted(self.local_experts)
        ea.in_device_ids, ea.out_device_ids = args.in_device_ids, args.out_device_ids
        ea.out_channel_infos = [C.ChannelInfo([tuple(x) for x in e], a, d) for e, a, d in args.out_channel_infos]
        ea.in_nccl_ids, ea.out_nccl_ids = args.in_nccl_ids, args.out_nccl_ids
        ea.attn_peer = args.attn_peer
        parts = {}
        for l in ea.attn_layer_ids:
            if l == 0:
                parts[l] = 0
            else:
                parts[l] = 1 if cfg.is_dense_layer(l - 1) else cfg.top_k + 1
        ea.parts_needed = parts
        ea.num_dp_groups = max(1, cfg.dp_size)
        ea.device = str(self.device)
        self.handles = C.init_engine_colocate(ea) if (self.has_attn and self.has_expert) else C.init_engine(ea)
        if self.hosts_head:
            self.handles.attn_pool.set_unordered_layer(L)
        if self.has_attn:
            self.handles.attn_scheduler.set_max_batch_size(cfg.max_batch_size_attn)
        if self.has_expert:
            self.handles.scheduler.set_max_batch_size(cfg.max_batch_size_expert)
        self._build_executor(attn_layers)

    def _init_tp_group(self, args: InitCoreArgs) -> None:
        """One process group per attention TP group (gloo on CPU, NCCL on GPUs) for the driver's batch broadcast and
        the o_proj all-reduce (reference: engine.py:253-256, where the TP group is a ``torch.distributed`` group too)."""
        import torch.distributed as dist
        from ..models import distributed as D
        assert not dist.is_initialized(), "attention TP needs one worker process per device"
        backend = "nccl" if self.device.type == "cuda" else "gloo"
        kw = {"device_id": self.device} if backend == "nccl" else {}
        dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{args.tp_master_port}", rank=self.tp_rank,
                                world_size=self.tp_size, **kw)
        D.set_tensor_model_parallel_config(self.model_config.clone(tp_size=self.tp_size, rank=self.tp_rank))
        self._dist = dist

    def _build_executor(self, attn_layers: List[int]) -> None:
        cfg, dev, dt = self.model_config, self.device, self.dtype
        sd = None
        if self.args.state_dict_path:
            sd = W.load_state_dict(self.args.state_dict_path)
        for l in attn_layers:
            m = MoEAttention(cfg, l, getattr(self, "tp_size", 1), getattr(self, "tp_rank", 0), device=dev, dtype=dt)
            m.load_weights(sd) if sd is not None else m.init_weights()
            self.attn_layers[l] = m
        for l, experts in self.local_experts.items():
            experts.sort()
            assert experts == list(range(experts[0], experts[-1] + 1)), "a worker holds a contiguous expert range"
            # --serial-gemm: one dense GEMM per expert instead of the grouped GEMM (the reference's non-grouped mode)
            cls = MoEExperts if cfg.enable_grouped_gemm else MoEExpertsSerial
            e = cls(cfg, l, experts[0], experts[-1] + 1, device=dev, dtype=dt,
                    max_batch_size=cfg.max_batch_size_expert if dev.type == "cuda" else 0)
            e.load_weights(sd) if sd is not None else e.init_weights()
            self.expert_layers[l] = e
        if self.has_attn:
            names = ["embed_tokens.weight", "norm.weight", "lm_head.weight"]
            g = sd if sd is not None else W.init_state_dict(cfg, dev, dt, names)
            self.embed_w = g["embed_tokens.weight"].to(device=dev, dtype=dt).contiguous()
            self.norm_w = g["norm.weight"].to(device=dev, dtype=dt)
            self.lm_head_w = g["lm_head.weight"].to(device=dev, dtype=dt).contiguous()
            cc = self.cache_config
            nb = cc.num_gpu_blocks or 1024
            self.block_size = cc.block_size
            kvh = next(iter(self.attn_layers.values())).num_kv_heads if self.attn_layers else cfg.num_kv_heads
            self.kv_cache = {l: torch.zeros(2, nb, cc.block_size, kvh, cfg.head_dim, dtype=dt, device=dev)
                             for l in attn_layers}
            self.block_mgr = C.BlockManager(cc.block_size, nb - cc.num_reserved_blocks, cc.num_reserved_blocks, 0)
            self.max_blocks = (cfg.max_seq_len + cc.block_size - 1) // cc.block_size
            self.graph_attn = None
            if cfg.enable_cuda_graph_attn and dev.type == "cuda" and getattr(self, "tp_size", 1) == 1 and attn_layers:
                # decode-only attention batches replay one CUDA graph per (layer, batch-size bucket), captured on
                # first use (reference: disagmoe/frontend/engine.py:325-383, disagmoe/executor/executor.py:118-347)
                from ..executor.executor import CUDAGraphAttnExecutor
                self.graph_attn = CUDAGraphAttnExecutor(cfg, cc, _EngineLayers(self, attn_layers))
                self.graph_attn.create_cuda_graph_buffers()
                self.graph_steps = 0

    # ---- loop -----------------------------------------------------------------------------------------------
    def start(self) -> None:
        C.start_engine(self.handles)
        self.end_flag = False
        target = self.attn_worker_loop if (self.tp_size > 1 and self.tp_rank > 0) else self._loop
        self.loop_thread = threading.Thread(target=target, daemon=True, name=f"engine-loop-{self.device_id}")
        self.loop_thread.start()

    def _loop(self) -> None:
        C.recorder_create(f"engine@{self.device_id}")
        try:
            while not self.end_flag:
                did = False
                if self.has_attn:
                    self.timer.start("schedule")
                    b = self.handles.attn_scheduler.schedule()
                    if b.metadata is not None:
                        t_sched = self.timer.stop("schedule")
                        self._timed_step(lambda: self.process_batch_attn(b), b.metadata.layer_id,
                                         b.metadata.num_tokens(), t_sched, self.handles.attn_scheduler)
                        did = True
                if self.has_expert:
                    self.timer.start("schedule")
                    tb = self.handles.scheduler.schedule()
                    if tb.metadata is not None:
                        t_sched = self.timer.stop("schedule")
                        self._timed_step(lambda: self.process_batch_expert(tb), tb.metadata.layer_id,
                                         tb.metadata.num_tokens(), t_sched, self.handles.scheduler)
                        did = True
                if not did:
                    # blocks without the GIL until tokens are queued (or 20 ms pass)
                    if self.has_attn:
                        self.handles.attn_scheduler.wait_for_new_requests(5 if self.has_expert else 20)
                    if self.has_expert:
                        self.handles.scheduler.wait_for_new_requests(5 if self.has_attn else 20)
        except Exception as e:   # surfaced through check_error(); the worker stays up for diagnosis
            import traceback
            self.error = traceback.format_exc()
            self._logger.error(self.error)

    # ---- attention TP (host-scheduled path) ----------------------------------------------------------------------
    def _tp_broadcast_batch(self, layer: int, token_ids, parts, meta: AttnMeta) -> None:
        """Driver -> workers of its TP group: what it is about to run (layer, token ids or partial rows, positions,
        slots, block table of the batch), as one pickled header and one tensor broadcast."""
        from ..models.utils import broadcast_pyobj
        dev = "cpu" if self.device.type == "cpu" else self.device
        hdr = dict(layer=layer, token_ids=token_ids, shape=None if parts is None else tuple(parts.shape),
                   pos=meta.positions.tolist(), slots=meta.slots.tolist(), table=meta.block_tables.tolist(),
                   bt_row=meta.bt_row.tolist(), ctx=meta.ctx_len.tolist(), n_prefill=meta.num_prefill_tokens,
                   n_decode=meta.num_decode_tokens, max_ctx=meta.max_ctx)
        broadcast_pyobj(hdr, 0, device=dev)
        if parts is not None:
            self._dist.broadcast(parts.contiguous(), 0)

    def attn_worker_loop(self) -> None:
        """Loop of a TP worker (a non-driver rank of an attention TP group): it takes no part in the token flow, it
        runs what the driver broadcasts on its own head shard and KV shard; the all-reduce inside the layer makes
        every rank hold the full result, and only the driver routes and dispatches it (reference:
        engine.py:538-612,757-772, asserted off there)."""
        from ..models.utils import broadcast_pyobj
        dev = self.device
        pdev = "cpu" if dev.type == "cpu" else dev
        t = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt).to(dev)
        try:
            while True:
                hdr = broadcast_pyobj(None, 0, device=pdev)
                if hdr.get("stop"):
                    return
                layer = hdr["layer"]
                resid = parts = None
                if hdr["token_ids"] is not None:
                    resid = F.embed(t(hdr["token_ids"]), self.embed_w)
                else:
                    parts = torch.empty(hdr["shape"], dtype=self.dtype, device=dev)
                    self._dist.broadcast(parts, 0)
                    resid = parts[:, 0].contiguous()
                    parts = parts[:, 1:] if parts.shape[1] > 1 else None
                meta = AttnMeta(t(hdr["pos"]), t(hdr["slots"], torch.int64), t(hdr["table"]), t(hdr["bt_row"]),
                                t(hdr["ctx"]), num_prefill_tokens=hdr["n_prefill"], num_decode_tokens=hdr["n_decode"],
                                max_ctx=hdr["max_ctx"])
                self.attn_layers[layer].forward(resid, parts, (self.kv_cache[layer][0], self.kv_cache[layer][1]), meta)
                self.metric.step()
        except Exception:
            import traceback
            self.error = traceback.format_exc()
            self._logger.error(self.error)

    # names of the reference's loops (engine.py:832-904): one loop serves both kinds of worker here
    def single_module_loop(self) -> None:
        self._loop()

    def dual_module_loop(self) -> None:
        self._loop()

    def _timed_step(self, fn, layer_id, n_tokens, t_sched, sched) -> None:
        self._queueing_delays.append(sched.get_cur_queueing_delay())
        t0 = time_ms()
        self.timer.start("step")
        with nvtx_range("engine.step"):
            fn()
        t_step = self.timer.stop("step")
        self.metric.step()
        self.metric.update("t_schedule", t_sched)
        self.metric.update("t_step", t_step)
        self.metric.update("effective_tokens", n_tokens)
        for name in ("preprocess", "execute", "postprocess"):
            v = self.timer.get(name)
            if v is not None:
                self.metric.update("t_" + name, v)
        if self.model_config.enable_trace:
            snap = sched.get_pool_snapshot()
            self.metric.update("queueing_tokens", float(sum(snap)))
            self.step_infos.append(StepInfo(t0, time_ms(), n_tokens, layer_id, layer_id,
                                            {i: v for i, v in enumerate(snap)}, threading.get_ident(), os.getpid()))

    # ---- attention role -------------------------------------------------------------------------------------
    def _attn_meta(self, m) -> AttnMeta:
        """Block-table bookkeeping for the batch (every row grows its sequence so that its position has a slot) and
        the device-side attention metadata."""
        bm = self.block_mgr
        seqs, pos = m.seq_ids, m.positions
        rows_of: Dict[int, int] = {}
        slots, bt_row = [], []
        for s, p, plen in zip(seqs, pos, m.init_prefill_lens):
            if not bm.has_seq_block_list(s):
                bm.allocate(s, max(plen, p + 1))
            bm.append_tokens(s, p, 1)
        for s, p in zip(seqs, pos):
            slots.append(bm.slot_of(s, p))
            bt_row.append(rows_of.setdefault(s, len(rows_of)))
        width = max(len(bm.get_seq_block_list(s)) for s in rows_of)
        table = torch.zeros(len(rows_of), width, dtype=torch.int32)
        for s, r in rows_of.items():
            bl = bm.get_seq_block_list(s)
            table[r, :len(bl)] = torch.tensor(bl, dtype=torch.int32)
        dev = self.device
        t = lambda x, dt=torch.int32: torch.tensor(x, dtype=dt).to(dev)
        return AttnMeta(t(pos), t(slots, torch.int64), table.to(dev), t(bt_row), t([p + 1 for p in pos]),
                        num_prefill_tokens=m.num_prefill_tokens, num_decode_tokens=m.num_decode_tokens,
                        max_ctx=max(pos) + 1)

    def graph_attention_steps(self) -> int:
        return int(getattr(self, "graph_steps", 0))

    def process_batch_attn(self, batch) -> None:
        cfg = self.model_config
        m = batch.metadata
        L = cfg.num_layers
        layer = m.layer_id
        n = m.num_tokens()
        self.timer.start("preprocess")
        if batch.data is None:
            ids = torch.tensor(m.token_ids, dtype=torch.int32).to(self.device)
            resid, parts = F.embed(ids, self.embed_w), None
        else:
            resid, parts = None, batch.data
        if layer == L:
            self.timer.stop("preprocess")
            return self._head_step(m, parts)
        meta = self._attn_meta(m)
        if self.tp_size > 1:
            self._tp_broadcast_batch(layer, list(m.token_ids) if batch.data is None else None, parts, meta)
        self.timer.stop("preprocess")
        self.timer.start("execute")
        if resid is None:
            # the first partial row doubles as the residual buffer that the layer updates in place
            resid = parts[:, 0].contiguous()
            parts = parts[:, 1:] if parts.shape[1] > 1 else None
        ga = getattr(self, "graph_attn", None)
        if ga is not None and m.num_prefill_tokens == 0 and ga.fits(n) and self.attn_layers[layer].weighted_router is None:
            from ..models.attention import AttnOutput
            y, tw, ti, r = ga.run(layer, meta.positions, resid, meta, parts)
            # the outputs alias the graph's static buffers: the dispatcher keeps rows beyond the next replay
            out = AttnOutput(None if y is None else y.clone(), r.clone(), tw, ti)
            self.graph_steps += 1
        else:
            out = self.attn_layers[layer].forward(resid, parts, (self.kv_cache[layer][0], self.kv_cache[layer][1]), meta)
        self.timer.stop("execute")
        self.timer.start("postprocess")
        keep = list(range(n))
        if layer == L - 1:
            # only rows whose logits are needed go on: decode rows and the last token of every prompt
            keep = [i for i in range(n) if m.init_prefill_lens[i] < 0 or m.positions[i] == m.init_prefill_lens[i] - 1]
        base = m.to_metadata()
        sel = base if len(keep) == n else base.at(keep)
        idx = None if len(keep) == n else torch.tensor(keep, dtype=torch.long, device=self.device)
        resid_rows = out.residual if idx is None else out.residual.index_select(0, idx)
        k = cfg.top_k
        dispatcher = self.handles.attn_dispatcher
        if out.expert_input is not None and len(keep) > 0:
            y = out.expert_input if idx is None else out.expert_input.index_select(0, idx)
            ids_l = (out.topk_ids if idx is None else out.topk_ids.index_select(0, idx)).reshape(-1).tolist()
            w_l = (out.topk_weights if idx is None else out.topk_weights.index_select(0, idx)).reshape(-1).tolist()
            em = C.Metadata.deserialize(sel.serialize())
            em.duplicate_topk(k)                      # token-major: row i*k + j is slot j of token i
            em.exp_ids, em.topk_weights = ids_l, w_l
            order = sorted(range(len(ids_l)), key=lambda i: ids_l[i])     # stable sort by expert id
            em = em.at(order)
            em.layer_id = layer
            rows = y.index_select(0, torch.tensor([i // k for i in order], dtype=torch.long, device=self.device))
            em.shape = [rows.shape[0], rows.shape[1]]
            em.dtype = "fp32" if rows.dtype == torch.float32 else "bf16"
            dispatcher.put(C.TensorBatch(rows.contiguous(), em), 0)
        if len(keep) > 0:
            rm = C.Metadata.deserialize(sel.serialize())
            rm.layer_id = layer + 1
            rm.exp_ids = [-1] * len(keep)
            rm.topk_slots = [0 if out.expert_input is None else k] * len(keep)
            rm.shape = [resid_rows.shape[0], resid_rows.shape[1]]
            rm.dtype = "fp32" if resid_rows.dtype == torch.float32 else "bf16"
            dispatcher.put(C.TensorBatch(resid_rows.contiguous(), rm), 1)
        self.timer.stop("postprocess")

    def _head_step(self, m, parts) -> None:
        cfg = self.model_config
        resid = parts[:, 0].contiguous()
        rest = parts[:, 1:] if parts.shape[1] > 1 else None
        _, h = F.add_rmsnorm(resid, rest, self.norm_w, cfg.rms_norm_eps, resid_out=resid)
        logits = gemm.linear(h, self.lm_head_w, out_dtype=torch.float32)
        ids = F.argmax(logits).tolist()
        if self.args.keep_logits:
            lc = logits.float().cpu()
            for i, (s, p) in enumerate(zip(m.seq_ids, m.positions)):
                self.logits_log[(s, p)] = lc[i]
        sm = m.to_metadata()
        sm.token_ids = ids
        sm.shape = [len(ids), 0]
        self.handles.attn_dispatcher.put(_id_batch(sm), 2)

    # ---- expert role ----------------------------------------------------------------------------------------
    def process_batch_expert(self, batch) -> None:
        cfg = self.model_config
        meta = batch.metadata
        layer = meta.layer_id
        self.timer.start("preprocess")
        experts = self.local_experts[layer]
        offs = torch.tensor(meta.get_expert_offsets(cfg.num_experts, experts), dtype=torch.int32).to(self.device)
        n = meta.num_tokens()
        self.timer.stop("preprocess")
        self.timer.start("execute")
        out = self.expert_layers[layer].forward(n, batch.data, offs)
        w = torch.tensor(meta.topk_weights, dtype=torch.float32).to(self.device)
        out = (out.float() * w[:, None]).to(out.dtype)
        self.timer.stop("execute")
        self.timer.start("postprocess")
        mapping = meta.sort_by_prefill_order()      # rows grouped by the attention replica that owns them
        inv = [0] * n
        for old, new in enumerate(mapping):
            inv[new] = old
        out = out.index_select(0, torch.tensor(inv, dtype=torch.long, device=self.device))
        meta.step_layer()
        self.handles.expert_dispatcher.put(C.TensorBatch(out.contiguous(), meta), 0)
        self.timer.stop("postprocess")

    # ---- control --------------------------------------------------------------------------------------------
    def release_seqs(self, seq_ids: List[int]) -> None:
        if self.block_mgr is not None:
            held = [s for s in seq_ids if self.block_mgr.has_seq_block_list(s)]
            self.block_mgr.batch_release(held)
            self.handles.attn_pool.release_seqs(seq_ids)

    def fetch_queueing_delays(self) -> List[float]:
        """Milliseconds the oldest row of every executed batch had waited in this worker's pool (reference:
        engine.py:919-920, where the underlying measurement is disabled)."""
        return list(self._queueing_delays)

    def set_device_id(self, device_id: int) -> None:
        self.device_id = device_id

    def get_node_ip(self) -> str:
        from ..utils.utils import get_ip
        return get_ip()

    @property
    def is_attn_driver(self) -> bool:
        return self.has_attn and self.model_config.tp_size > 1 and self.model_config.rank == 0

    @property
    def is_attn_worker(self) -> bool:
        return self.has_attn and self.model_config.tp_size > 1 and self.model_config.rank > 0

    def get_configured_kv_cache_blocks(self) -> int:
        return self.cache_config.num_gpu_blocks

    def determine_kv_cache_blocks(self, gpu_memory_utilization: float = 0.9) -> int:
        """Paged-KV blocks that fit next to the weights already resident: (total * utilisation - used) / bytes of
        one block over this worker's attention layers (reference: engine.py:328-348; no profile run is needed here
        because the activation buffers of a step are a few MB)."""
        cfg, cc = self.model_config, self.cache_config
        n_layers = max(1, len(self.attn_layers))
        kvh = next(iter(self.attn_layers.values())).num_kv_heads if self.attn_layers else cfg.num_kv_heads
        block_bytes = n_layers * 2 * cc.block_size * kvh * cfg.head_dim * torch.empty(0, dtype=self.dtype).element_size()
        if self.device.type != "cuda":
            return cc.num_gpu_blocks or 1024
        free, total = torch.cuda.mem_get_info(self.device)
        return max(0, int((total * gpu_memory_utilization - (total - free)) // block_bytes))

    def num_free_blocks(self) -> int:
        return self.block_mgr.num_free_blocks() if self.block_mgr is not None else 0

    def fetch_step_stats(self):
        infos, self.step_infos = self.step_infos, []
        traces = {k: [(t.msg, t.t_start, t.t_dur, t.track_id) for t in v] for k, v in C.recorder_output().items()}
        return infos, traces, self.metric

    def fetch_logits(self) -> Dict[Tuple[int, int], torch.Tensor]:
        out, self.logits_log = self.logits_log, {}
        return out

    def set_schedule_policy(self, policy: str) -> None:
        if self.has_attn:
            self.handles.attn_scheduler.set_schedule_policy(policy)
        if self.has_expert:
            self.handles.scheduler.set_schedule_policy(policy)

    def set_schedule_block(self, step: int) -> None:
        if self.has_attn:
            self.handles.attn_scheduler.set_schedule_block(step)
        if self.has_expert:
            self.handles.scheduler.set_schedule_block(step)

    def check_error(self) -> Optional[str]:
        """The engine loop's exception, or the one that ended a native helper thread (pool / dispatcher) of this worker."""
        return self.error or (C.helper_error() or None)

    def heartbeat(self) -> float:
        return time.time()

    def start_profile(self, profile_dir: Optional[str] = None) -> None:
        profile_dir = profile_dir or os.environ.get("DMOE_PROFILE_DIR") or None
        C.recorder_enable(True)
        self._torch_prof = None
        if profile_dir:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if self.device.type == "cuda":
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._torch_prof = torch.profiler.profile(
                activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(profile_dir))
            self._torch_prof.start()

    def stop_profile(self) -> None:
        if getattr(self, "_torch_prof", None) is not None:
            self._torch_prof.stop()
            self._torch_prof = None

    def reset(self) -> None:
        self.metric = Metric()
        self.step_infos = []
        self._queueing_delays = []

    def terminate(self) -> None:
        self.end_flag = True
        tp_worker = getattr(self, "tp_size", 1) > 1 and self.tp_rank > 0
        if self.loop_thread is not None and not tp_worker:      # a TP worker's loop waits for its driver's stop message
            self.loop_thread.join(timeout=10)
        if getattr(self, "tp_size", 1) > 1 and self.tp_rank == 0 and self.error is None:
            from ..models.utils import broadcast_pyobj
            try:
                broadcast_pyobj({"stop": True}, 0, device="cpu" if self.device.type == "cpu" else self.device)
            except Exception:
                pass
        if self.handles is not None:
            C.stop_engine(self.handles)


def _id_batch(meta):
    b = C.TensorBatch()
    b.metadata = meta
    return b


class TokenizerEngine:
    """Front door: turns a request into one row per prompt token and hands it to the native ``Tokenizer``."""

    def __init__(self, device_id: int, out_device_ids: List[int], attn_peer: Dict[int, int]):
        self.tokenizer = C.init_tokenizer(device_id, out_device_ids, attn_peer)
        self.t_submitted: Dict[int, float] = {}

    def start(self) -> None:
        self.tokenizer.start()

    def put_single_request(self, req_id: int, prompt_ids: List[int], dp_rank: int) -> None:
        self.t_submitted[req_id] = time.time()
        self.tokenizer.put_request(req_id, list(prompt_ids), dp_rank)

    def put_request(self, req_ids: List[int], prompts: List[List[int]], dp_ranks: List[int]) -> None:
        for r, p, d in zip(req_ids, prompts, dp_ranks):
            self.put_single_request(r, p, d)

    put_requests = put_request          # the reference's name (engine.py:1068)
    process_request = put_single_request

    def fetch_submitted_time(self) -> Dict[int, float]:
        return dict(self.t_submitted)

    def reset(self) -> None:
        self.t_submitted.clear()

    def terminate(self) -> None:
        self.tokenizer.terminate()


class SamplerEngine:
    """Bookkeeping end of the loop (output lengths, finish rule, SLO timestamps) around the native ``Sampler``."""

    def __init__(self, device_id: int, out_device_ids: List[int], attn_peer: Dict[int, int], min_output_len: int,
                 max_output_len: int, top_k: int = 1, ignore_eos: bool = True):
        self.sampler = C.init_sampler(device_id, min_output_len, max_output_len, top_k, out_device_ids, attn_peer,
                                      ignore_eos, False)

    def start(self) -> None:
        self.sampler.start_all()

    def set_request_output_len(self, req_id: int, n: int) -> None:
        self.sampler.set_request_output_len(req_id, n)

    def wait_for_n_requests(self, n_request: int, timeout: float = 600.0) -> Dict[int, SloStat]:
        """Blocks until ``n_request`` requests have finished; their SLO timestamps by request id (reference:
        engine.py:1035-1043)."""
        t0, out = time.time(), {}
        while len(out) < n_request:
            for s in self.sampler.fetch_finished_slo_stats():
                out[s.req_id] = SloStat.from_c(s)
            if time.time() - t0 > timeout:
                raise TimeoutError(f"{len(out)} of {n_request} requests finished within {timeout} s")
            if len(out) < n_request:
                time.sleep(0.002)
        return out

    def fetch_finished_results(self):
        return self.sampler.fetch_finished_slo_stats()

    def fetch_sampler_step_infos(self):
        return self.sampler.fetch_step_infos()

    def get_output_tokens(self, req_id: int) -> List[int]:
        return self.sampler.get_output_tokens(req_id)

    def num_finished(self) -> int:
        return self.sampler.num_finished()

    def reset(self) -> None:
        self.sampler.reset()

    def terminate(self) -> None:
        self.sampler.stop_all()
