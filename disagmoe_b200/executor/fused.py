"""Whole-iteration executor of a colocated worker: every layer's attention and experts on one device.

This is the one-GPU point of the throughput curve (the reference's ``ColocatePlacement`` + ``dual_module_loop``,
disagmoe/utils/placement.py:467-508, disagmoe/frontend/engine.py:873-904), restructured for Blackwell: a decode
iteration is one chain of kernels with no host round trip between the router and the expert GEMMs (the expert
histogram, offsets, sort and token records stay on the device), captured in a CUDA graph per batch-size bucket.

    embed -> L x [ add+RMSNorm -> QKV (tcgen05) -> RoPE + KV append -> paged attention -> o_proj + residual
                   -> RMSNorm + gate + top-k -> sort-by-expert dispatch -> grouped GEMM-1 + SwiGLU
                   -> grouped GEMM-2 with combine epilogue (router weight, un-permute) ]
          -> add+RMSNorm -> LM head -> argmax

The same code runs on CPU tensors (fp32) through the PyTorch restatements of the ops, which is how it is checked
against the oracle without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config import CacheConfig, ModelConfig
from ..models import weights as W
from ..models.attention import AttnMeta, MoEAttention
from ..models.experts import MoEExperts
from ..ops import _lib
from ..ops import functional as F
from ..ops import gemm
from ..utils.utils import get_graph_batch_size, graph_batch_sizes


class StepBuffers:
    """Static activation buffers for up to ``cap`` tokens (CUDA graphs replay on fixed addresses)."""

    def __init__(self, cfg: ModelConfig, cap: int, device, dtype, max_blocks: int, q_size: int, kv_size: int):
        H, k, E = cfg.hidden_size, cfg.top_k, cfg.num_experts
        self.cap = cap
        z = lambda *s, dt=dtype: torch.zeros(*s, dtype=dt, device=device)
        self.ids = z(cap, dt=torch.int32)
        self.positions = z(cap, dt=torch.int32)
        self.slots = z(cap, dt=torch.int64)
        self.ctx_len = z(cap, dt=torch.int32)
        self.bt_row = z(cap, dt=torch.int32)
        self.resid = z(cap, H)
        self.parts = z(cap, k, H)
        self.dispatch = F.DispatchBuffers(cap * k, H, E, device, dtype)
        self.parts_base = torch.tensor([self.parts.data_ptr()], dtype=torch.int64, device=device)
        self.next_ids = z(cap, dt=torch.int32)
        self.logits = z(cap, cfg.vocab_size, dt=torch.float32)
        # prompt segments of the current step for the tiled causal attention kernel (filled by prefill())
        self.prefill_tiles = z(cap, 4, dt=torch.int32)
        self.ctx_len_decode = z(cap, dt=torch.int32)
        self.n_prefill_tiles = 0


class FusedModelExecutor:
    def __init__(self, cfg: ModelConfig, cache_cfg: CacheConfig, device="cuda", dtype: Optional[torch.dtype] = None,
                 max_batch_size: int = 256, max_prefill_tokens: int = 4096, state_dict: Optional[W.StateDict] = None,
                 num_blocks: Optional[int] = None, enable_cuda_graph: bool = True, layer_ids: Optional[List[int]] = None):
        self.cfg, self.cache_cfg = cfg, cache_cfg
        self.device = torch.device(device)
        self.dtype = dtype or cfg.dtype
        self.block_size = cache_cfg.block_size
        self.max_batch_size = max_batch_size
        self.max_blocks_per_seq = (cfg.max_seq_len + self.block_size - 1) // self.block_size
        self.layer_ids = list(range(cfg.num_layers)) if layer_ids is None else layer_ids
        self.enable_cuda_graph = enable_cuda_graph and self.device.type == "cuda"
        self.attn: Dict[int, MoEAttention] = {}
        self.experts: Dict[int, MoEExperts] = {}
        for l in self.layer_ids:
            a = MoEAttention(cfg, l, device=self.device, dtype=self.dtype)
            a.load_weights(state_dict) if state_dict is not None else a.init_weights()
            self.attn[l] = a
            if not cfg.is_dense_layer(l):
                e = MoEExperts(cfg, l, device=self.device, dtype=self.dtype)
                e.load_weights(state_dict) if state_dict is not None else e.init_weights()
                self.experts[l] = e
        names = ["embed_tokens.weight", "norm.weight", "lm_head.weight"]
        sd = state_dict if state_dict is not None else W.init_state_dict(cfg, self.device, self.dtype, names)
        self.embed_w = sd["embed_tokens.weight"].to(device=self.device, dtype=self.dtype).contiguous()
        self.norm_w = sd["norm.weight"].to(device=self.device, dtype=self.dtype)
        self.lm_head_w = sd["lm_head.weight"].to(device=self.device, dtype=self.dtype).contiguous()

        self.num_blocks = num_blocks or cache_cfg.num_gpu_blocks or self._profile_num_blocks()
        kv_heads = self.attn[self.layer_ids[0]].num_kv_heads
        # [layers, 2, num_blocks, block_size, kv_heads, head_dim] (reference: disagmoe/executor/executor.py:81-83)
        self.kv_cache = torch.zeros(len(self.layer_ids), 2, self.num_blocks, self.block_size, kv_heads, cfg.head_dim,
                                    dtype=self.dtype, device=self.device)
        self.block_tables = torch.zeros(max_batch_size, self.max_blocks_per_seq, dtype=torch.int32, device=self.device)
        a0 = self.attn[self.layer_ids[0]]
        self.decode_buf = StepBuffers(cfg, max_batch_size, self.device, self.dtype, self.max_blocks_per_seq, a0.q_size,
                                      a0.kv_size)
        self.prefill_buf = StepBuffers(cfg, max_prefill_tokens, self.device, self.dtype, self.max_blocks_per_seq,
                                       a0.q_size, a0.kv_size) if max_prefill_tokens > max_batch_size else self.decode_buf
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_sizes: List[int] = []
        self.graph_launches: Dict[int, int] = {}

    # ---- memory -------------------------------------------------------------------------------------------------
    def _profile_num_blocks(self) -> int:
        cfg = self.cfg
        per_block = len(self.layer_ids) * 2 * self.block_size * self.attn[self.layer_ids[0]].num_kv_heads * cfg.head_dim * \
            torch.empty((), dtype=self.dtype).element_size()
        if self.device.type != "cuda":
            return 512
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - (1.0 - self.cache_cfg.gpu_memory_utilization) * total - (6 << 30)
        return max(64, int(budget // per_block))

    def kv_of(self, local_idx: int):
        return self.kv_cache[local_idx, 0], self.kv_cache[local_idx, 1]

    # ---- one iteration -------------------------------------------------------------------------------------------
    def _forward(self, buf: StepBuffers, T: int, max_ctx: int, want_logits: bool):
        cfg = self.cfg
        meta = AttnMeta(buf.positions[:T], buf.slots[:T], self.block_tables, buf.bt_row[:T], buf.ctx_len[:T],
                        max_ctx=max_ctx, prefill_tiles=buf.prefill_tiles, n_prefill_tiles=buf.n_prefill_tiles,
                        ctx_len_decode=buf.ctx_len_decode[:T])
        resid = buf.resid[:T]
        F.embed(buf.ids[:T], self.embed_w, out=resid)
        parts = None
        d = buf.dispatch
        for i, l in enumerate(self.layer_ids):
            a = self.attn[l]
            a.counts = d.counts
            out = a.forward(resid, parts, self.kv_of(i), meta)   # updates `resid` in place
            if out.expert_input is None:
                parts = None
                continue
            F.dispatch_local(out.expert_input, out.topk_ids, out.topk_weights, d)
            n = T * cfg.top_k
            if resid.is_cuda:
                self.experts[l].forward_combine(n, d.xs[:n], d.offs, d.recs[:n], buf.parts_base, cfg.hidden_size)
            else:
                self.experts[l].forward_combine(n, d.xs[:n], d.offs, d.recs[:n], None, cfg.hidden_size,
                                                outs=[buf.parts.view(-1, cfg.hidden_size)])
            parts = buf.parts[:T]
        _, h = F.add_rmsnorm(resid, parts, self.norm_w, cfg.rms_norm_eps, resid_out=resid)
        logits = gemm.linear(h, self.lm_head_w, out=buf.logits[:T], out_dtype=torch.float32)
        F.argmax(logits, out=buf.next_ids[:T])
        return buf.next_ids[:T], (logits if want_logits else None)

    def _fill(self, buf, T, ids, positions, slots, ctx_len, bt_row):
        nb = self.device.type == "cuda"
        buf.ids[:T].copy_(ids, non_blocking=nb)
        buf.positions[:T].copy_(positions, non_blocking=nb)
        buf.slots[:T].copy_(slots, non_blocking=nb)
        buf.ctx_len[:T].copy_(ctx_len, non_blocking=nb)
        buf.bt_row[:T].copy_(bt_row, non_blocking=nb)

    def set_block_table_row(self, row: int, blocks: List[int]) -> None:
        t = torch.tensor(blocks, dtype=torch.int32)
        self.block_tables[row, :len(blocks)].copy_(t)

    def prefill(self, ids, positions, slots, ctx_len, bt_row, want_logits=False):
        """Eager pass over prompt tokens (any number of sequences packed together). Host tensors in, device out."""
        T = ids.shape[0]
        assert T <= self.prefill_buf.cap, f"{T} prefill tokens exceed the buffer ({self.prefill_buf.cap})"
        buf = self.prefill_buf
        self._fill(buf, T, ids, positions, slots, ctx_len, bt_row)
        buf.n_prefill_tiles = 0
        if self.device.type == "cuda":
            a0 = self.attn[self.layer_ids[0]]
            tiles, covered = F.build_prefill_tiles(bt_row, positions, F.prefill_tile_tokens(a0.num_heads, a0.num_kv_heads))
            if len(tiles):
                buf.n_prefill_tiles = len(tiles)
                buf.prefill_tiles[:len(tiles)].copy_(tiles, non_blocking=True)
                cd = torch.as_tensor(ctx_len).clone()
                cd[covered] = 0
                buf.ctx_len_decode[:T].copy_(cd, non_blocking=True)
        try:
            return self._forward(buf, T, int(ctx_len.max()), want_logits)
        finally:
            buf.n_prefill_tiles = 0      # the decode path (and its CUDA graphs) shares the buffers when they are one object

    def capture(self, sizes: Optional[List[int]] = None) -> None:
        """Warm-up (compiles nothing, but sizes scratch buffers and sets kernel attributes) and graph capture."""
        if not self.enable_cuda_graph:
            return
        sizes = sizes or graph_batch_sizes(self.max_batch_size, self.cfg.graph_stride * 4)
        buf = self.decode_buf
        buf.ctx_len.fill_(1)
        buf.slots.fill_(-1)
        side = torch.cuda.Stream(self.device)
        for b in sorted(set(sizes), reverse=True):
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._forward(buf, b, self.cfg.max_seq_len, False)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = _lib.LAUNCHES
            with torch.cuda.graph(g):
                self._forward(buf, b, self.cfg.max_seq_len, False)
            self.graphs[b] = g
            self.graph_launches[b] = _lib.LAUNCHES - n0
        self.graph_sizes = sorted(self.graphs)
        torch.cuda.synchronize()

    def decode(self, ids, positions, slots, ctx_len, bt_row=None, want_logits=False):
        """One decode iteration for B sequences (one token each). Inputs are host (pinned) or device tensors of
        length B; returns the device tensor of greedy next-token ids (and logits when asked)."""
        B = ids.shape[0]
        buf = self.decode_buf
        if bt_row is None:
            bt_row = torch.arange(B, dtype=torch.int32)
        if self.graph_sizes and not want_logits and B <= self.graph_sizes[-1]:
            _, b = get_graph_batch_size(B, self.graph_sizes)
            self._fill(buf, B, ids, positions, slots, ctx_len, bt_row)
            if b > B:
                # padding rows: no KV append, attend to nothing
                buf.slots[B:b].fill_(-1)
                buf.ctx_len[B:b].fill_(0)
                buf.ids[B:b].fill_(0)
            self.graphs[b].replay()
            _lib.add_launches(self.graph_launches[b])
            return buf.next_ids[:B], None
        self._fill(buf, B, ids, positions, slots, ctx_len, bt_row)
        return self._forward(buf, B, int(ctx_len.max()) if not ctx_len.is_cuda else self.cfg.max_seq_len, want_logits)
