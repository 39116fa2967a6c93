"""Tensor-parallel helpers of the attention group (reference: disagmoe/models/distributed.py:16-59).

Three all-reduce back ends, chosen per call site: the native ``NcclGroupChannel`` (``set_tensor_model_parallel_channel``),
``torch.distributed`` (NCCL on GPUs, gloo on CPU), and -- on the fused path -- the peer-memory one-shot reduction that
is folded into the kernel consuming the o_proj output (:mod:`disagmoe_b200.parallel.tp`).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from ..config import ModelConfig

_tp_model_config: Optional[ModelConfig] = None
_channel = None
_group = None


def set_tensor_model_parallel_config(model_config: ModelConfig) -> None:
    global _tp_model_config
    _tp_model_config = model_config


def set_tensor_model_parallel_channel(channel) -> None:
    global _channel
    _channel = channel


def set_tensor_model_parallel_group(group) -> None:
    global _group
    _group = group


def get_tensor_model_parallel_rank() -> int:
    return _tp_model_config.rank if _tp_model_config is not None else 0


def get_tensor_model_parallel_world_size() -> int:
    return _tp_model_config.tp_size if _tp_model_config is not None else 1


def tensor_model_parallel_all_reduce(tensor: Tensor, group=None) -> Tensor:
    if get_tensor_model_parallel_world_size() == 1 and group is None:
        return tensor
    if not tensor.is_contiguous():
        tensor = tensor.contiguous()
    if _channel is not None and tensor.is_cuda and (_tp_model_config is None or _tp_model_config.tp_enable_inter_group):
        _channel.all_reduce(tensor)
        _channel.sync()
    else:
        dist.all_reduce(tensor, group=group or _group)
    return tensor


def group_sync() -> None:
    if _channel is not None:
        _channel.barrier()
    elif dist.is_initialized():
        dist.barrier(group=_group)


def tensor_model_parallel_all_gather(tensor: Tensor, dim: int = -1, group=None) -> Tensor:
    world = dist.get_world_size(group or _group) if dist.is_initialized() else 1
    if world == 1:
        return tensor
    parts = [torch.empty_like(tensor) for _ in range(world)]
    dist.all_gather(parts, tensor.contiguous(), group=group or _group)
    return torch.cat(parts, dim=dim)
