"""Per-layer executors (reference: disagmoe/executor/executor.py:22-389).

``AttnExecutor``           one ``MoEAttention`` per local layer + the paged KV cache
                           ``[layers, 2, num_blocks, block_size, kv_heads, head_dim]``
``CUDAGraphAttnExecutor``  static input buffers and one captured graph per (layer, batch-size bucket); buckets follow
                           ``[1] + range(max(stride, ep), max_bs + 1, stride)``
``ExpertsExecutor``        one ``MoEExperts`` per local layer (grouped GEMM, or one GEMM per expert with
                           ``enable_grouped_gemm = False``)
``ParallelAttnExecutor``   attention executor of one tensor-parallel rank
"""
from __future__ import annotations

from enum import Enum
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor

from ..config import CacheConfig, ModelConfig
from ..models.attention import AttnMeta, AttnOutput, MoEAttention
from ..models.experts import MoEExperts, MoEExpertsSerial
from ..utils.utils import get_graph_batch_size, graph_batch_sizes


class ExecutorType(Enum):
    ATTENTION_EXEC = 1
    EXPERTS_EXEC = 2


class Executor:
    def __init__(self, model_config: ModelConfig, device="cuda", dtype=None):
        self.model_config = model_config
        self.device = torch.device(device)
        self.dtype = dtype or model_config.dtype
        self.layer_ids = model_config.layer_ids if model_config.layer_ids is not None else \
            list(range(model_config.num_layers))
        self.layer_mappings = {l: i for i, l in enumerate(self.layer_ids)}   # global -> local

    def initialize_cache(self, num_blocks: int) -> None:
        raise NotImplementedError


class AttnExecutor(Executor):
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, device="cuda", dtype=None, state_dict=None,
                 tp_size: int = 1, tp_rank: int = 0, tp_group=None):
        super().__init__(model_config, device, dtype)
        self.cache_config = cache_config
        self.type = ExecutorType.ATTENTION_EXEC
        self.operators: List[MoEAttention] = []
        for l in self.layer_ids:
            m = MoEAttention(model_config, l, tp_size, tp_rank, device=self.device, dtype=self.dtype, tp_group=tp_group)
            m.load_weights(state_dict) if state_dict is not None else m.init_weights()
            self.operators.append(m)
        self.cache = None

    def initialize_cache(self, num_blocks: int) -> None:
        cfg, cc = self.model_config, self.cache_config
        kvh = self.operators[0].num_kv_heads
        self.cache = torch.zeros(len(self.layer_ids), 2, num_blocks, cc.block_size, kvh, cfg.head_dim, dtype=self.dtype,
                                 device=self.device)

    def kv(self, layer_id: int):
        c = self.cache[self.layer_mappings[layer_id]]
        return c[0], c[1]

    def execute(self, layer_id: int, positions: Tensor, hidden_states: Tensor, attn_metadata: AttnMeta,
                parts: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor]:
        """Returns (expert input rows, top-k weights, top-k ids); ``hidden_states`` is the residual stream and is
        updated in place."""
        attn_metadata.positions = positions
        out: AttnOutput = self.operators[self.layer_mappings[layer_id]].forward(hidden_states, parts, self.kv(layer_id),
                                                                                attn_metadata)
        return out.expert_input, out.topk_weights, out.topk_ids

    def profile_execute(self, batch_size: int) -> None:
        """One dummy decode step per layer at ``batch_size`` (used to find the memory high-water mark)."""
        cfg = self.model_config
        if self.cache is None:
            self.initialize_cache(max(2, batch_size // self.cache_config.block_size + 2))
        i32 = lambda x: torch.full((batch_size,), x, dtype=torch.int32, device=self.device)
        meta = AttnMeta(i32(0), torch.full((batch_size,), -1, dtype=torch.int64, device=self.device),
                        torch.zeros(batch_size, 1, dtype=torch.int32, device=self.device), None, i32(1), max_ctx=1)
        x = torch.zeros(batch_size, cfg.hidden_size, dtype=self.dtype, device=self.device)
        for l in self.layer_ids:
            self.execute(l, meta.positions, x, meta)

    @staticmethod
    def build(model_config: ModelConfig, cache_config: CacheConfig, **kw) -> "AttnExecutor":
        if model_config.tp_size > 1:
            return ParallelAttnExecutor(model_config, cache_config, **kw)
        return AttnExecutor(model_config, cache_config, **kw)


class ParallelAttnExecutor(AttnExecutor):
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, **kw):
        kw.setdefault("tp_size", model_config.tp_size)
        kw.setdefault("tp_rank", model_config.rank)
        super().__init__(model_config, cache_config, **kw)


class CUDAGraphAttnExecutor:
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, attn_executor: AttnExecutor):
        self.model_config, self.cache_config, self.attn_executor = model_config, cache_config, attn_executor
        self.max_batch_size = model_config.max_batch_size_attn
        self.graph_batch_sizes = graph_batch_sizes(self.max_batch_size, model_config.graph_stride, model_config.ep_size)
        self.graphs: Dict[Tuple[int, int, int], torch.cuda.CUDAGraph] = {}      # (layer, bucket, partial rows)
        self.outputs: Dict[Tuple[int, int, int], Tuple[Tensor, Tensor, Tensor]] = {}
        self.static_parts: Optional[Tensor] = None

    def create_cuda_graph_buffers(self) -> None:
        cfg, dev, B = self.model_config, self.attn_executor.device, self.max_batch_size
        max_blocks = (cfg.max_seq_len + self.cache_config.block_size - 1) // self.cache_config.block_size
        self.static_input = torch.zeros(B, cfg.hidden_size, dtype=self.attn_executor.dtype, device=dev)
        self.static_positions = torch.zeros(B, dtype=torch.int32, device=dev)
        self.static_slots = torch.full((B,), -1, dtype=torch.int64, device=dev)
        self.static_ctx = torch.zeros(B, dtype=torch.int32, device=dev)
        self.static_block_table = torch.zeros(B, max_blocks, dtype=torch.int32, device=dev)

    def _meta(self, b: int) -> AttnMeta:
        return AttnMeta(self.static_positions[:b], self.static_slots[:b], self.static_block_table, None,
                        self.static_ctx[:b], num_decode_tokens=b, max_ctx=self.model_config.max_seq_len)

    def _capture_one(self, l: int, b: int, P: int) -> None:
        """Warm-up and capture of layer l at batch bucket b with P partial rows per token added to the residual."""
        ex = self.attn_executor
        if P > 0 and (self.static_parts is None or self.static_parts.shape[1] < P):
            self.static_parts = torch.zeros(self.max_batch_size, P, self.model_config.hidden_size,
                                            dtype=self.attn_executor.dtype, device=self.attn_executor.device)
        parts = self.static_parts[:b, :P] if P > 0 else None
        meta = self._meta(b)
        side = torch.cuda.Stream(ex.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ex.execute(l, meta.positions, self.static_input[:b], meta, parts)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = ex.execute(l, meta.positions, self.static_input[:b], meta, parts)
        self.graphs[(l, b, P)] = g
        self.outputs[(l, b, P)] = out

    def capture(self) -> None:
        """Captures every (layer, bucket) graph up front for batches that carry no partial rows; graphs for batches
        with partial rows (top-k expert outputs + carried residual) are captured the first time they are needed."""
        for l in self.attn_executor.layer_ids:
            for b in self.graph_batch_sizes:
                self._capture_one(l, b, 0)
        torch.cuda.synchronize()

    def fits(self, n: int) -> bool:
        return 0 < n <= self.graph_batch_sizes[-1]

    def run(self, layer_id: int, positions: Tensor, hidden_states: Tensor, meta: AttnMeta,
            parts: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
        """Copies the inputs into the static buffers, replays the bucket's graph; returns (expert input, weights, ids,
        residual) views of the first ``n`` rows (None where the layer has no router). The views alias static buffers
        that the next replay of the same graph overwrites."""
        n = hidden_states.shape[0]
        _, b = get_graph_batch_size(n, self.graph_batch_sizes)
        P = 0 if parts is None else parts.shape[1]
        # capture warm-ups run the layer for real: slots = -1 and ctx = 0 keep them away from the KV cache
        self.static_slots[:b].fill_(-1)
        self.static_ctx[:b].fill_(0)
        if (layer_id, b, P) not in self.graphs:
            self._capture_one(layer_id, b, P)
        self.static_input[:n].copy_(hidden_states)
        if P > 0:
            self.static_parts[:n, :P].copy_(parts)
        self.static_positions[:n].copy_(positions)
        self.static_slots[:n].copy_(meta.slots)
        self.static_ctx[:n].copy_(meta.ctx_len)
        rows = meta.bt_row.long() if meta.bt_row is not None else torch.arange(n, device=hidden_states.device)
        w = meta.block_tables.shape[1]
        self.static_block_table[:n, :w].copy_(meta.block_tables.index_select(0, rows))
        self.graphs[(layer_id, b, P)].replay()
        y, tw, ti = self.outputs[(layer_id, b, P)]
        cut = lambda t: None if t is None else t[:n]
        return cut(y), cut(tw), cut(ti), self.static_input[:n]


class ExpertsExecutor(Executor):
    def __init__(self, model_config: ModelConfig, device="cuda", dtype=None, state_dict=None, e_lo: int = 0,
                 e_hi: Optional[int] = None):
        super().__init__(model_config, device, dtype)
        self.type = ExecutorType.EXPERTS_EXEC
        cls = MoEExperts if model_config.enable_grouped_gemm else MoEExpertsSerial
        e_hi = e_hi if e_hi is not None else e_lo + model_config.num_experts_per_rank
        self.operators: List[MoEExperts] = []
        for l in self.layer_ids:
            m = cls(model_config, l, e_lo, e_hi, device=self.device, dtype=self.dtype,
                    max_batch_size=model_config.max_batch_size_expert)
            m.load_weights(state_dict) if state_dict is not None else m.init_weights()
            self.operators.append(m)

    def execute(self, layer_id: int, num_tokens: int, hidden_states: Tensor, batch_sizes: Tensor) -> Tensor:
        """``batch_sizes`` are the per-local-expert row counts (int tensor on any device) of the expert-sorted rows."""
        offs = torch.zeros(batch_sizes.numel() + 1, dtype=torch.int32, device=hidden_states.device)
        offs[1:] = batch_sizes.to(hidden_states.device).cumsum(0).int()
        return self.operators[self.layer_mappings[layer_id]].forward(num_tokens, hidden_states, offs)
