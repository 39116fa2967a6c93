"""The attention half of a decoder layer as the attention workers run it.

pre-norm -> QKV -> RoPE + paged KV append -> paged attention -> o_proj (+ residual) -> post-norm -> router top-k,
plus what stays on the attention side of the disaggregation: shared experts and dense FFN layers. Counterpart of
``MoEAttention`` (disagmoe/models/attention.py:76-233); differences: real router logits instead of
``torch.rand_like``, the residual stream is kept (the reference drops it at attention.py:221,233), positions are
real, and every op is one of this package's kernels (CUDA) or its PyTorch restatement (CPU / fp32).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..config import ModelConfig
from ..ops import functional as F
from ..ops import gemm
from . import weights as W


@dataclass
class AttnMeta:
    """Per-batch attention metadata (the role of FlashAttentionMetadata built at disagmoe/frontend/engine.py:429-485).

    positions [T] int32: absolute position of every token; slots [T] int64: flat KV slot (block * block_size +
    offset) the token's K/V is appended to; block_tables [R, max_blocks] int32; bt_row [T] int32: block-table row of
    the token's sequence (None = identity); ctx_len [T] int32: tokens each query attends to (position + 1).
    """
    positions: torch.Tensor
    slots: torch.Tensor
    block_tables: torch.Tensor
    bt_row: Optional[torch.Tensor]
    ctx_len: torch.Tensor
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    max_ctx: int = 0
    # prompt segments for the tiled causal kernel (CUDA only): device int32 [>= n_prefill_tiles, 4] from
    # ops.functional.build_prefill_tiles, and ctx_len with the covered rows set to 0 for the per-token kernel
    prefill_tiles: Optional[torch.Tensor] = None
    n_prefill_tiles: int = 0
    ctx_len_decode: Optional[torch.Tensor] = None


@dataclass
class AttnOutput:
    expert_input: Optional[torch.Tensor]   # normalised rows the routed experts consume (None for a dense layer)
    residual: torch.Tensor                 # residual stream after attention (+ shared experts / dense FFN)
    topk_weights: Optional[torch.Tensor]
    topk_ids: Optional[torch.Tensor]


class MoEAttention(torch.nn.Module):
    def __init__(self, cfg: ModelConfig, layer_id: int, tp_size: int = 1, tp_rank: int = 0, device="cpu",
                 dtype: Optional[torch.dtype] = None, tp_group=None):
        super().__init__()
        self.cfg, self.layer_id, self.tp_size, self.tp_rank, self.tp_group = cfg, layer_id, tp_size, tp_rank, tp_group
        self.dtype = dtype or cfg.dtype
        self.device = torch.device(device)
        assert cfg.num_heads % tp_size == 0
        self.num_heads = cfg.num_heads // tp_size
        self.num_kv_heads = W.kv_heads_per_rank(cfg, tp_size)
        self.head_dim = cfg.head_dim
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.is_dense = cfg.is_dense_layer(layer_id)
        # expert popularity for trace-weighted routing: set from the file named by DMOE_WEIGHTED_ROUTER_FILE
        self.weighted_router: Optional[torch.Tensor] = None if self.is_dense else self._load_weighted_router()
        self._gen: Optional[torch.Generator] = None
        self.counts: Optional[torch.Tensor] = None            # device histogram fed to the dispatch kernel
        self.route_bias: Optional[torch.Tensor] = None        # fp32 [E] added to the gate logits (popularity skew)

    def _load_weighted_router(self) -> Optional[torch.Tensor]:
        """Per-expert popularity of this layer from a routing trace (reference: attention.py:169-182). The file is a
        CSV with a ``layer_id`` column, optionally a ``category`` column (DMOE_WEIGHTED_ROUTER_CATEGORY, default
        ``closed_qa``), and one count column per expert as its last ``num_experts`` columns; the rows of this layer are
        summed and normalised. With it set, the router samples expert ids from the popularity vector instead of
        using the gate (synthetic load studies); ``use_popularity_as_logit_bias`` keeps the gate and skews it."""
        import os
        path = os.environ.get("DMOE_WEIGHTED_ROUTER_FILE", "")
        if not path:
            return None
        assert os.path.exists(path), f"weighted router file {path} does not exist"
        import pandas as pd
        df = pd.read_csv(path)
        if "category" in df.columns:
            df = df[df["category"] == os.environ.get("DMOE_WEIGHTED_ROUTER_CATEGORY", "closed_qa")]
        df = df[df["layer_id"] == self.layer_id]
        counts = torch.tensor(df.iloc[:, -self.cfg.num_experts:].to_numpy(dtype="float64")).sum(0)
        assert counts.numel() == self.cfg.num_experts and float(counts.sum()) > 0, "no trace rows for this layer"
        return (counts / counts.sum()).float()

    def use_popularity_as_logit_bias(self) -> None:
        """Turns the loaded popularity vector into a device-side logit bias (log popularity): the gate still decides,
        skewed towards the popular experts, and routing stays on the device (usable inside CUDA graphs)."""
        if self.weighted_router is not None:
            self.route_bias = torch.log(self.weighted_router.clamp_min(1e-6)).float().to(self.device)
            self.weighted_router = None

    # ---- weights ------------------------------------------------------------------------------------------
    def param_names(self):
        p = f"layers.{self.layer_id}."
        names = [p + "qkv_proj.weight", p + "o_proj.weight", p + "pre_attention_layernorm.weight",
                 p + "post_attention_layernorm.weight"]
        cfg = self.cfg
        if self.is_dense:
            names += [p + "mlp.w13_weight", p + "mlp.w2_weight"]
        else:
            names.append(p + "gate.weight")
            if cfg.num_shared_experts > 0:
                names += [p + "shared_expert.w13_weight", p + "shared_expert.w2_weight"]
                if cfg.shared_expert_gate:
                    names.append(p + "shared_expert_gate.weight")
        return names

    def load_weights(self, sd: W.StateDict) -> None:
        cfg, p = self.cfg, f"layers.{self.layer_id}."
        to = dict(device=self.device, dtype=self.dtype)
        self.qkv_w = W.shard_qkv(sd[p + "qkv_proj.weight"], cfg, self.tp_size, self.tp_rank).to(**to).contiguous()
        self.o_w = W.shard_o_proj(sd[p + "o_proj.weight"], cfg, self.tp_size, self.tp_rank).to(**to).contiguous()
        self.pre_ln = sd[p + "pre_attention_layernorm.weight"].to(**to)
        self.post_ln = sd[p + "post_attention_layernorm.weight"].to(**to)
        self.gate_w = self.shared_w13 = self.shared_w2 = self.shared_gate = self.mlp_w13 = self.mlp_w2 = None
        if self.is_dense:
            self.mlp_w13, self.mlp_w2 = (t.to(**to) for t in
                                         W.to_runtime_expert_layout(sd[p + "mlp.w13_weight"], sd[p + "mlp.w2_weight"]))
            return
        self.gate_w = sd[p + "gate.weight"].to(**to).contiguous()
        if cfg.num_shared_experts > 0:
            self.shared_w13, self.shared_w2 = (t.to(**to) for t in W.to_runtime_expert_layout(
                sd[p + "shared_expert.w13_weight"], sd[p + "shared_expert.w2_weight"]))
            if cfg.shared_expert_gate:
                self.shared_gate = sd[p + "shared_expert_gate.weight"].to(**to).contiguous()

    def init_weights(self, device=None) -> None:
        """Seeded random weights created directly on the target device (only this layer's tensors)."""
        dev = device or self.device
        self.load_weights(W.init_state_dict(self.cfg, device=dev, dtype=self.dtype, names=self.param_names()))

    # ---- forward ------------------------------------------------------------------------------------------
    def _tp_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            from .distributed import tensor_model_parallel_all_reduce
            return tensor_model_parallel_all_reduce(x, self.tp_group)
        return x

    def _ffn(self, h, w13, w2, residual):
        act = gemm.swiglu_linear(h, w13)
        return gemm.linear(act, w2, residual=residual, out=residual)

    def attention(self, resid: Optional[torch.Tensor], parts: Optional[torch.Tensor], kv_cache, meta: AttnMeta
                  ) -> torch.Tensor:
        """Everything up to and including o_proj + residual. ``parts`` [T, P, H] are added to ``resid`` first (the
        partial expert outputs and the carried residual of the previous layer)."""
        cfg = self.cfg
        # the residual stream is updated in place: `resid` is owned by the caller's step buffers
        resid, h = F.add_rmsnorm(resid, parts, self.pre_ln, cfg.rms_norm_eps, resid_out=resid)
        kc, vc = kv_cache
        if h.is_cuda:
            # RoPE and the paged K / V append run in the QKV GEMM's epilogue (only the q columns of `qkv` are written)
            table = gemm.rope_table(cfg.max_seq_len, self.head_dim, cfg.rope_theta, h.device)   # positions < max_seq_len
            rope = gemm.RopeAppend(table, meta.positions, meta.slots, kc, vc, self.num_heads, self.num_kv_heads,
                                   self.head_dim)
            qkv = gemm.linear(h, self.qkv_w, comm=gemm.GemmComm(rope=rope))
        else:
            qkv = gemm.linear(h, self.qkv_w)
            F.rope_kv_append(qkv, meta.positions, meta.slots, kc, vc, self.num_heads, self.num_kv_heads,
                             self.head_dim, cfg.rope_theta)
        T = qkv.shape[0]
        splits = 1
        if qkv.is_cuda:
            splits = F.pick_attn_splits(T, self.num_kv_heads, meta.max_ctx or cfg.max_seq_len, kc.shape[1])
        tiled = qkv.is_cuda and meta.n_prefill_tiles > 0
        attn = F.paged_attention(qkv[:, :self.q_size], kc, vc, meta.block_tables, meta.bt_row,
                                 meta.ctx_len_decode if tiled else meta.ctx_len,
                                 self.num_heads, self.num_kv_heads, self.head_dim, splits=splits)
        if tiled:
            # prompt segments: one pass over the sequence's K / V per tile of 64 query rows instead of one per row
            F.prefill_attention(qkv[:, :self.q_size], kc, vc, meta.block_tables, meta.prefill_tiles,
                                meta.n_prefill_tiles, self.num_heads, self.num_kv_heads, self.head_dim, attn)
        if self.tp_size == 1:
            return gemm.linear(attn, self.o_w, residual=resid, out=resid)
        part = self._tp_reduce(gemm.linear(attn, self.o_w))
        resid.copy_((part.float() + resid.float()).to(resid.dtype))
        return resid

    def route(self, resid2: torch.Tensor, want_logits: bool = False):
        cfg = self.cfg
        y, ids, w, logits = F.route(resid2, self.post_ln, cfg.rms_norm_eps, self.gate_w, cfg.top_k, cfg.norm_topk_prob,
                                    counts=self.counts if resid2.is_cuda else None, want_logits=want_logits,
                                    logit_bias=self.route_bias)
        if self.weighted_router is not None:
            ids, w = self._random_routing_with_weights(resid2.shape[0], resid2.device)
        return y, ids, w, logits

    def set_route_skew(self, zipf_alpha: float) -> None:
        """Skews expert popularity towards a Zipf(alpha) distribution over expert ids (expert 0 the most popular) by
        adding log-popularity to the gate logits; alpha = 0 removes the skew. Stays on the device (graph-capturable),
        unlike the trace-weighted sampling below."""
        if self.is_dense:
            return
        if zipf_alpha <= 0:
            self.route_bias = None
            return
        E = self.cfg.num_experts
        pop = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** zipf_alpha
        self.route_bias = torch.log(pop / pop.sum()).float().to(self.device)

    def shared_experts(self, y: torch.Tensor, resid: torch.Tensor) -> torch.Tensor:
        """resid += shared_expert(y) (times sigmoid(y . g) for a gated shared expert), in place."""
        if self.shared_w13 is None:
            return resid
        if self.shared_gate is None:
            return self._ffn(y, self.shared_w13, self.shared_w2, resid)
        sh = self._ffn(y, self.shared_w13, self.shared_w2, None)
        g = torch.sigmoid(y.float() @ self.shared_gate.float().T)
        resid.copy_((resid.float() + sh.float() * g).to(resid.dtype))
        return resid

    def dense_ffn(self, resid: torch.Tensor, h: Optional[torch.Tensor] = None) -> torch.Tensor:
        """resid += mlp(rmsnorm(resid)) for a layer with a dense FFN, in place (h: the normalised rows if the
        caller already has them)."""
        if h is None:
            h = F.rmsnorm(resid, self.post_ln, self.cfg.rms_norm_eps)
        return self._ffn(h, self.mlp_w13, self.mlp_w2, resid)

    def _random_routing_with_weights(self, T: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """Trace-weighted routing: expert ids sampled without replacement from a popularity vector
        (reference: attention.py:52-74,184-190)."""
        if self._gen is None:
            self._gen = torch.Generator(device="cpu")
            self._gen.manual_seed(self.cfg.seed * 1000 + self.layer_id)
        pop = self.weighted_router.float().cpu()
        probs = pop.expand(T, -1)
        ids = torch.multinomial(probs, self.cfg.top_k, replacement=False, generator=self._gen)
        w = torch.gather(probs, 1, ids)
        w = w / w.sum(1, keepdim=True)
        return ids.int().to(device), w.float().to(device)

    def forward(self, resid: Optional[torch.Tensor], parts: Optional[torch.Tensor], kv_cache, meta: AttnMeta,
                want_logits: bool = False) -> AttnOutput:
        cfg = self.cfg
        resid2 = self.attention(resid, parts, kv_cache, meta)
        if self.is_dense:
            return AttnOutput(None, self.dense_ffn(resid2), None, None)
        y, ids, w, logits = self.route(resid2, want_logits)
        resid2 = self.shared_experts(y, resid2)
        out = AttnOutput(y, resid2, w, ids)
        out.router_logits = logits
        return out
