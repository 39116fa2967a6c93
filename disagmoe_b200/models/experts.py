"""The expert half of a decoder layer as the expert workers run it: grouped SwiGLU FFN over the local experts.

Counterpart of ``MoEExperts`` / ``MoEExpertsSerial`` (disagmoe/models/experts.py:9-119). Input rows are sorted by
local expert; ``offs`` [E_local + 1] are the row offsets of the experts (device tensor: the host never needs the
counts). Weights are held K-contiguous: ``w13 [E_local, 2I, H]`` (gate rows then up rows), ``w2 [E_local, H, I]``.
GEMM-1 runs with the SiLU-and-mul epilogue fused; GEMM-2 either writes plain rows or runs the combine epilogue
(router-weight scale + scatter to the token's owner).

On a GPU the grouped path keeps both stacks tile by tile (``ops.gemm.block_weight``: every 128 x 64 box the GEMM
fetches is 16 KB of consecutive addresses), which streams the weights 6-8 % faster than row-major stacks at decode
sizes; ``w_blocked`` says so, and ``logical_weights()`` returns row-major copies for anything that is not the GEMM.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..config import ModelConfig
from ..ops import gemm
from . import weights as W


class MoEExperts(torch.nn.Module):
    def __init__(self, cfg: ModelConfig, layer_id: int, e_lo: int = 0, e_hi: Optional[int] = None, device="cpu",
                 dtype: Optional[torch.dtype] = None, max_batch_size: int = 0):
        super().__init__()
        self.cfg, self.layer_id = cfg, layer_id
        self.e_lo, self.e_hi = e_lo, cfg.num_experts if e_hi is None else e_hi
        self.num_experts = self.e_hi - self.e_lo
        self.hidden_size, self.intermediate_size = cfg.hidden_size, cfg.intermediate_size
        self.device, self.dtype = torch.device(device), dtype or cfg.dtype
        self.w_blocked = False
        self.cache_up = self.cache_down = None
        if max_batch_size > 0 and self.device.type == "cuda":
            # persistent activation buffers (the role of cache_up / cache_down at experts.py:57-58)
            self.cache_up = torch.empty(max_batch_size, self.intermediate_size, dtype=self.dtype, device=self.device)
            self.cache_down = torch.empty(max_batch_size, self.hidden_size, dtype=self.dtype, device=self.device)

    def param_names(self):
        p = f"layers.{self.layer_id}.experts."
        return [p + "w13_weight", p + "w2_weight"]

    def load_weights(self, sd: W.StateDict) -> None:
        p = f"layers.{self.layer_id}.experts."
        w13 = W.shard_experts(sd[p + "w13_weight"], self.e_lo, self.e_hi)
        w2 = W.shard_experts(sd[p + "w2_weight"], self.e_lo, self.e_hi)
        w13, w2 = W.to_runtime_expert_layout(w13, w2)
        self.w13_weight = w13.to(device=self.device, dtype=self.dtype).contiguous()
        self.w2_weight = w2.to(device=self.device, dtype=self.dtype).contiguous()
        if self._want_blocked():
            self.w13_weight = gemm.block_weight(self.w13_weight)      # one stack at a time: the peak is one extra copy
            self.w2_weight = gemm.block_weight(self.w2_weight)
            self.w_blocked = True

    def _want_blocked(self) -> bool:
        """Tile-blocked stacks: grouped path on a GPU, whole 128 x 64 tiles in both stacks."""
        H, I = self.hidden_size, self.intermediate_size
        return (self.device.type == "cuda" and type(self) is MoEExperts and I % 128 == 0 and H % 128 == 0 and
                os.environ.get("DMOE_BLOCKED_WEIGHTS", "1") != "0")

    def logical_weights(self):
        """(w13 [E, 2I, H], w2 [E, H, I]) in row-major order, whatever order the GEMM copies are kept in."""
        if not self.w_blocked:
            return self.w13_weight, self.w2_weight
        return gemm.unblock_weight(self.w13_weight), gemm.unblock_weight(self.w2_weight)

    def init_weights(self) -> None:
        """Seeded random weights created on the target device expert by expert (no copy of the multi-GB stacked
        tensor is ever made) and transposed into the runtime layout. The values equal
        ``load_weights(init_state_dict(cfg))`` for a state dict drawn on the same kind of device."""
        cfg, H, I = self.cfg, self.hidden_size, self.intermediate_size
        E = self.num_experts
        self.w13_weight = torch.empty(E, 2 * I, H, dtype=self.dtype, device=self.device)
        self.w2_weight = torch.empty(E, H, I, dtype=self.dtype, device=self.device)
        blocked = self._want_blocked()
        for i, e in enumerate(range(self.e_lo, self.e_hi)):
            w13, w2 = W.init_expert(cfg, self.layer_id, e, self.device, self.dtype)
            self.w13_weight[i].copy_(gemm.block_weight(w13.T.contiguous()) if blocked else w13.T)
            self.w2_weight[i].copy_(gemm.block_weight(w2.T.contiguous()) if blocked else w2.T)
        self.w_blocked = blocked

    def forward(self, bs: int, hiddens: torch.Tensor, offs: torch.Tensor, out: Optional[torch.Tensor] = None
                ) -> torch.Tensor:
        """hiddens [bs, H] sorted by local expert, offs [E_local + 1] -> [bs, H]."""
        up_buf = self.cache_up[:bs] if self.cache_up is not None and bs <= self.cache_up.shape[0] else None
        if out is None and self.cache_down is not None and bs <= self.cache_down.shape[0]:
            out = self.cache_down[:bs]
        act = gemm.grouped_swiglu(hiddens, self.w13_weight, offs, out=up_buf, w_blocked=self.w_blocked)
        return gemm.grouped_linear(act, self.w2_weight, offs, out=out, w_blocked=self.w_blocked)

    def forward_combine(self, bs: int, hiddens: torch.Tensor, offs: torch.Tensor, recs: torch.Tensor,
                        bases: torch.Tensor, ld_out: int, outs=None) -> None:
        """Same FFN, but GEMM-2 scales every row by its router weight and scatters it to its owner (combine)."""
        up_buf = self.cache_up[:bs] if self.cache_up is not None and bs <= self.cache_up.shape[0] else None
        act = gemm.grouped_swiglu(hiddens, self.w13_weight, offs, out=up_buf, w_blocked=self.w_blocked)
        gemm.grouped_combine(act, self.w2_weight, offs, recs, bases, ld_out, outs=outs, w_blocked=self.w_blocked)


class MoEExpertsSerial(MoEExperts):
    """One expert at a time through the dense GEMM entry points (the reference's non-grouped mode)."""

    def forward(self, bs: int, hiddens: torch.Tensor, offs: torch.Tensor, out: Optional[torch.Tensor] = None
                ) -> torch.Tensor:
        bounds = offs.tolist()
        if out is None:
            out = torch.empty(bs, self.hidden_size, dtype=hiddens.dtype, device=hiddens.device)
        for e in range(self.num_experts):
            a, b = bounds[e], bounds[e + 1]
            if b > a:
                act = gemm.swiglu_linear(hiddens[a:b], self.w13_weight[e])
                gemm.linear(act, self.w2_weight[e], out=out[a:b])
        return out
