"""Checkpoint layout, seeded random initialisation, sharding and save / load.

Checkpoint ("state dict") names and shapes follow the reference's parameters:

    layers.{l}.qkv_proj.weight                 [(h + 2 kv) * hd, H]   q | k | v row blocks   (disagmoe/models/linear.py:626-712)
    layers.{l}.o_proj.weight                   [H, h * hd]                                   (linear.py:967-1014)
    layers.{l}.gate.weight                     [E, H]                                        (disagmoe/models/attention.py:159-164)
    layers.{l}.pre_attention_layernorm.weight  [H]
    layers.{l}.post_attention_layernorm.weight [H]                                           (attention.py:166-167)
    layers.{l}.experts.w13_weight              [E, H, 2 I]   gate half then up half, [in, out] (disagmoe/models/experts.py:42-55)
    layers.{l}.experts.w2_weight               [E, I, H]

plus what a real model needs and the reference mocks away: ``embed_tokens.weight [V, H]``, ``norm.weight [H]``,
``lm_head.weight [V, H]``, shared experts ``layers.{l}.shared_expert.{w13_weight [H, 2 Is], w2_weight [Is, H]}``,
``layers.{l}.shared_expert_gate.weight [1, H]`` and dense FFN layers ``layers.{l}.mlp.{w13_weight, w2_weight}``.

Sharding rules are those of the reference's weight loaders: q heads and kv heads are split over TP ranks (kv heads
replicated when tp > kv heads, linear.py:672-678), o_proj is split along its input dimension (linear.py:1016-1051),
expert tensors are sliced ``[e_lo:e_hi]`` per EP rank.

The kernels want every GEMM weight K-contiguous ("[out, in]"), so expert weights are transposed once at load time
into the runtime layout ``w13 [E, 2 I, H]`` / ``w2 [E, H, I]`` (:func:`to_runtime_expert_layout`).
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..config import ModelConfig

StateDict = Dict[str, torch.Tensor]


def param_shapes(cfg: ModelConfig) -> Dict[str, Tuple[int, ...]]:
    H, hd = cfg.hidden_size, cfg.head_dim
    shapes: Dict[str, Tuple[int, ...]] = {
        "embed_tokens.weight": (cfg.vocab_size, H),
        "norm.weight": (H,),
        "lm_head.weight": (cfg.vocab_size, H),
    }
    for l in range(cfg.num_layers):
        p = f"layers.{l}."
        shapes[p + "qkv_proj.weight"] = ((cfg.num_heads + 2 * cfg.num_kv_heads) * hd, H)
        shapes[p + "o_proj.weight"] = (H, cfg.num_heads * hd)
        shapes[p + "pre_attention_layernorm.weight"] = (H,)
        shapes[p + "post_attention_layernorm.weight"] = (H,)
        if cfg.is_dense_layer(l):
            shapes[p + "mlp.w13_weight"] = (H, 2 * cfg.dense_intermediate_size)
            shapes[p + "mlp.w2_weight"] = (cfg.dense_intermediate_size, H)
            continue
        shapes[p + "gate.weight"] = (cfg.num_experts, H)
        shapes[p + "experts.w13_weight"] = (cfg.num_experts, H, 2 * cfg.intermediate_size)
        shapes[p + "experts.w2_weight"] = (cfg.num_experts, cfg.intermediate_size, H)
        if cfg.num_shared_experts > 0:
            shapes[p + "shared_expert.w13_weight"] = (H, 2 * cfg.shared_intermediate_size)
            shapes[p + "shared_expert.w2_weight"] = (cfg.shared_intermediate_size, H)
            if cfg.shared_expert_gate:
                shapes[p + "shared_expert_gate.weight"] = (1, H)
    return shapes


def _name_seed(seed: int, name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return (h ^ (seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF


def is_expert_stack(name: str) -> bool:
    return name.endswith(".experts.w13_weight") or name.endswith(".experts.w2_weight")


def init_tensor(cfg: ModelConfig, name: str, shape: Tuple[int, ...], device="cpu", dtype=None) -> torch.Tensor:
    """One parameter, N(0, init_std) (norm weights = 1), drawn from a generator seeded by (cfg.seed, name): the
    value of a tensor does not depend on which other tensors a process creates, so every worker can materialise
    only its shard's names and still agree with a single-process model. The stacked expert tensors are drawn expert
    by expert from (cfg.seed, name + "." + expert index), so an expert-parallel worker that creates only its own
    experts (:func:`init_expert`) gets exactly the slices of the full tensor. Draws on a CUDA device come from a
    different generator than CPU draws: compare models initialised on the same kind of device."""
    dtype = dtype or cfg.dtype
    if name.endswith("layernorm.weight") or name == "norm.weight":
        return torch.ones(shape, dtype=dtype, device=device)
    if is_expert_stack(name) and len(shape) == 3:
        return torch.stack([init_tensor(cfg, f"{name}.{e}", tuple(shape[1:]), device, dtype) for e in range(shape[0])])
    gen = torch.Generator(device=device)
    gen.manual_seed(_name_seed(cfg.seed, name))
    t = torch.empty(shape, dtype=torch.float32 if torch.device(device).type == "cpu" else dtype, device=device)
    t.normal_(0.0, cfg.init_std, generator=gen)
    return t.to(dtype)


def init_expert(cfg: ModelConfig, layer_id: int, e: int, device="cpu", dtype=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Checkpoint-layout (w13 [H, 2I], w2 [I, H]) weights of global expert ``e`` of layer ``layer_id``: the same values
    as ``init_state_dict(cfg)["layers.<l>.experts.w13_weight"][e]`` / ``w2_weight[e]`` on the same kind of device."""
    p = f"layers.{layer_id}.experts."
    H, I = cfg.hidden_size, cfg.intermediate_size
    return (init_tensor(cfg, f"{p}w13_weight.{e}", (H, 2 * I), device, dtype),
            init_tensor(cfg, f"{p}w2_weight.{e}", (I, H), device, dtype))


def init_state_dict(cfg: ModelConfig, device="cpu", dtype=None, names: Optional[Iterable[str]] = None) -> StateDict:
    shapes = param_shapes(cfg)
    names = list(names) if names is not None else list(shapes)
    return {n: init_tensor(cfg, n, shapes[n], device, dtype) for n in names}


# ---------------------------------------------------------------------------------------------- sharding
def kv_heads_per_rank(cfg: ModelConfig, tp: int) -> int:
    return max(1, cfg.num_kv_heads // tp)


def shard_qkv(w: torch.Tensor, cfg: ModelConfig, tp: int, rank: int) -> torch.Tensor:
    """Rows of the fused qkv weight that TP rank ``rank`` owns: its q heads, then its (possibly replicated) kv heads."""
    if tp == 1:
        return w
    hd, h, kv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    assert h % tp == 0 and (kv % tp == 0 or tp % kv == 0)
    hq = h // tp
    q = w[rank * hq * hd:(rank + 1) * hq * hd]
    kvr = kv_heads_per_rank(cfg, tp)
    kv_idx = rank * kvr if kv >= tp else rank // (tp // kv)
    k0 = h * hd
    k = w[k0 + kv_idx * hd:k0 + (kv_idx + kvr) * hd]
    v0 = k0 + kv * hd
    v = w[v0 + kv_idx * hd:v0 + (kv_idx + kvr) * hd]
    return torch.cat([q, k, v], dim=0).contiguous()


def shard_o_proj(w: torch.Tensor, cfg: ModelConfig, tp: int, rank: int) -> torch.Tensor:
    if tp == 1:
        return w
    per = cfg.num_heads // tp * cfg.head_dim
    return w[:, rank * per:(rank + 1) * per].contiguous()


def shard_experts(w: torch.Tensor, e_lo: int, e_hi: int) -> torch.Tensor:
    return w[e_lo:e_hi]


def to_runtime_expert_layout(w13_ckpt: torch.Tensor, w2_ckpt: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[.., H, 2I] / [.., I, H] ([in, out]) -> K-contiguous [.., 2I, H] / [.., H, I] ([out, in])."""
    return w13_ckpt.transpose(-1, -2).contiguous(), w2_ckpt.transpose(-1, -2).contiguous()


def to_checkpoint_expert_layout(w13_rt: torch.Tensor, w2_rt: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return w13_rt.transpose(-1, -2).contiguous(), w2_rt.transpose(-1, -2).contiguous()


# ---------------------------------------------------------------------------------------------- save / load
def save_state_dict(sd: StateDict, path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    tmp = path + ".tmp"
    torch.save({k: v.detach().cpu() for k, v in sd.items()}, tmp)
    os.replace(tmp, path)


def load_state_dict(path: str, device="cpu", dtype=None) -> StateDict:
    sd = torch.load(path, map_location="cpu", weights_only=True)
    return {k: v.to(device=device, dtype=dtype or v.dtype) for k, v in sd.items()}


def check_state_dict(cfg: ModelConfig, sd: StateDict) -> List[str]:
    """Names that are missing or have the wrong shape (empty list = compatible)."""
    bad = []
    for n, shp in param_shapes(cfg).items():
        if n not in sd or tuple(sd[n].shape) != tuple(shp):
            bad.append(n)
    return bad
