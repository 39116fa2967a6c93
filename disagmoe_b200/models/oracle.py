"""fp32 single-process oracle of the served model.

A dependency-light restatement of the real decoder: embedding -> [RMSNorm, QKV, neox RoPE, causal attention,
o_proj, residual, RMSNorm, softmax top-k router, SwiGLU experts (+ shared experts / dense FFN), weighted combine,
residual] x L -> final norm -> LM head -> greedy. It keeps a plain contiguous KV history per request (no paging,
no batching tricks) so that it shares no code with the engine it checks. Model math follows
disagmoe/models/attention.py:202-233 and disagmoe/models/experts.py:81-96 with the reference's mocked parts
(random router logits, dropped residual, constant positions) replaced by the real semantics.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

from ..config import ModelConfig
from .weights import StateDict


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, hd, theta):
    # x [T, n, hd]
    half = hd // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float32) * 2.0 / hd)
    ang = pos.float()[:, None] * inv[None]
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


class OracleModel:
    def __init__(self, cfg: ModelConfig, sd: StateDict):
        self.cfg = cfg
        self.sd = {k: v.detach().float().cpu() for k, v in sd.items()}
        self.kv: Dict[int, List[Tuple[torch.Tensor, torch.Tensor]]] = {}   # req -> per layer (K [S, kv, hd], V)
        self.routing_log: List[Tuple[int, torch.Tensor, torch.Tensor]] = []

    def release(self, req_id: int) -> None:
        self.kv.pop(req_id, None)

    def _ffn(self, x, w13, w2):
        """x [T, H]; w13 [H, 2I] ([in, out]), w2 [I, H]."""
        h = x @ w13
        I = h.shape[-1] // 2
        return (torch.nn.functional.silu(h[:, :I]) * h[:, I:]) @ w2

    def _layer(self, l: int, x: torch.Tensor, pos: torch.Tensor, req_id: int) -> torch.Tensor:
        cfg, sd, p = self.cfg, self.sd, f"layers.{l}."
        T, hd, h, kv = x.shape[0], cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        hn = _rms(x, sd[p + "pre_attention_layernorm.weight"], cfg.rms_norm_eps)
        qkv = hn @ sd[p + "qkv_proj.weight"].T
        q = _rope(qkv[:, :h * hd].view(T, h, hd), pos, hd, cfg.rope_theta)
        k = _rope(qkv[:, h * hd:(h + kv) * hd].view(T, kv, hd), pos, hd, cfg.rope_theta)
        v = qkv[:, (h + kv) * hd:].view(T, kv, hd)
        hist = self.kv.setdefault(req_id, [None] * cfg.num_layers)
        if hist[l] is None:
            K, V = k, v
        else:
            K, V = torch.cat([hist[l][0], k]), torch.cat([hist[l][1], v])
        hist[l] = (K, V)
        S = K.shape[0]
        g = h // kv
        Kh, Vh = K.repeat_interleave(g, dim=1), V.repeat_interleave(g, dim=1)     # [S, h, hd]
        scores = torch.einsum("thd,shd->hts", q, Kh) / math.sqrt(hd)
        key_pos = torch.arange(S)[None, None, :]
        mask = key_pos > pos[None, :, None]      # causal on absolute positions
        scores = scores.masked_fill(mask, float("-inf"))
        attn = torch.einsum("hts,shd->thd", torch.softmax(scores, -1), Vh).reshape(T, h * hd)
        x = x + attn @ sd[p + "o_proj.weight"].T
        hn2 = _rms(x, sd[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        if cfg.is_dense_layer(l):
            return x + self._ffn(hn2, sd[p + "mlp.w13_weight"], sd[p + "mlp.w2_weight"])
        logits = hn2 @ sd[p + "gate.weight"].T
        probs = torch.softmax(logits, -1)
        w, ids = torch.topk(probs, cfg.top_k, dim=-1)
        if cfg.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        self.routing_log.append((l, ids.clone(), w.clone()))
        out = torch.zeros_like(x)
        w13, w2 = sd[p + "experts.w13_weight"], sd[p + "experts.w2_weight"]
        for t in range(T):
            for j in range(cfg.top_k):
                e = int(ids[t, j])
                out[t] += w[t, j] * self._ffn(hn2[t:t + 1], w13[e], w2[e])[0]
        if cfg.num_shared_experts > 0:
            sh = self._ffn(hn2, sd[p + "shared_expert.w13_weight"], sd[p + "shared_expert.w2_weight"])
            if cfg.shared_expert_gate:
                sh = sh * torch.sigmoid(hn2 @ sd[p + "shared_expert_gate.weight"].T)
            out = out + sh
        return x + out

    @torch.no_grad()
    def forward(self, req_id: int, token_ids: List[int], start_pos: Optional[int] = None) -> torch.Tensor:
        """Runs the tokens of one request (a prompt, or one decode token); returns logits [T, V] (fp32)."""
        cfg, sd = self.cfg, self.sd
        if start_pos is None:
            hist = self.kv.get(req_id)
            start_pos = 0 if hist is None or hist[0] is None else hist[0][0].shape[0]
        ids = torch.tensor(token_ids, dtype=torch.long)
        pos = torch.arange(start_pos, start_pos + len(token_ids))
        x = sd["embed_tokens.weight"][ids]
        for l in range(cfg.num_layers):
            x = self._layer(l, x, pos, req_id)
        return _rms(x, sd["norm.weight"], cfg.rms_norm_eps) @ sd["lm_head.weight"].T

    @torch.no_grad()
    def generate(self, req_id: int, prompt: List[int], n_new: int) -> Tuple[List[int], torch.Tensor]:
        """Greedy decoding: returns (n_new generated ids, the logits row that produced each of them [n_new, V])."""
        logits = self.forward(req_id, prompt)[-1]
        out, rows = [], []
        for _ in range(n_new):
            rows.append(logits)
            tok = int(logits.argmax())
            out.append(tok)
            if len(out) == n_new:
                break
            logits = self.forward(req_id, [tok])[-1]
        return out, torch.stack(rows)
