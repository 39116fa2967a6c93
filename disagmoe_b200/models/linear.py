"""Linear layers with checkpoint loaders and TP sharding (reference: disagmoe/models/linear.py:139-1097, itself derived
from vLLM): ``ReplicatedLinear``, ``ColumnParallelLinear``, ``MergedColumnParallelLinear``, ``QKVParallelLinear``,
``RowParallelLinear``. Weights are ``[out, in]`` bf16; the forward pass is the tcgen05 GEMM of :mod:`disagmoe_b200.ops.gemm`
(or its PyTorch restatement on CPU). ``weight_loader(param, loaded_weight, shard_id)`` copies the slice of a full
checkpoint tensor that this TP rank owns, with the reference's rules: column-parallel layers split the output rows,
merged layers split every logical sub-matrix, the QKV layer splits q heads and kv heads (kv heads are replicated when
tp > kv heads), row-parallel layers split the input columns and all-reduce their output.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from ..ops import gemm
from .distributed import tensor_model_parallel_all_gather, tensor_model_parallel_all_reduce


class UnquantizedLinearMethod:
    """bf16 weights, no quantisation (the only method the reference instantiates)."""

    def create_weights(self, layer: nn.Module, in_features: int, out_features: int, params_dtype, device) -> None:
        w = nn.Parameter(torch.empty(out_features, in_features, dtype=params_dtype, device=device), requires_grad=False)
        layer.register_parameter("weight", w)

    def apply(self, layer: nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = gemm.linear(x, layer.weight)
        return y if bias is None else y + bias


class LinearBase(nn.Module):
    def __init__(self, input_size: int, output_size: int, params_dtype=None, device="cpu", prefix: str = ""):
        super().__init__()
        self.input_size, self.output_size, self.prefix = input_size, output_size, prefix
        self.params_dtype = params_dtype or torch.get_default_dtype()
        self.device_ = torch.device(device)
        self.quant_method = UnquantizedLinearMethod()
        self.bias = None

    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.weight.data.copy_(torch.empty(self.weight.shape).normal_(0, std, generator=g))


class ReplicatedLinear(LinearBase):
    def __init__(self, input_size, output_size, bias: bool = False, params_dtype=None, device="cpu", prefix=""):
        super().__init__(input_size, output_size, params_dtype, device, prefix)
        self.quant_method.create_weights(self, input_size, output_size, self.params_dtype, self.device_)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, shard_id=None) -> None:
        assert param.shape == loaded_weight.shape
        param.data.copy_(loaded_weight)

    def forward(self, x):
        return self.quant_method.apply(self, x, self.bias), None


class ColumnParallelLinear(LinearBase):
    """Y = X A^T with A split along its output rows: rank r holds rows [r * out/tp, (r+1) * out/tp)."""

    def __init__(self, input_size, output_size, bias: bool = False, gather_output: bool = False, tp_size: int = 1,
                 tp_rank: int = 0, params_dtype=None, device="cpu", prefix="", output_sizes: Optional[List[int]] = None):
        super().__init__(input_size, output_size, params_dtype, device, prefix)
        self.tp_size, self.tp_rank, self.gather_output = tp_size, tp_rank, gather_output
        assert output_size % tp_size == 0
        self.output_size_per_partition = output_size // tp_size
        self.output_sizes = output_sizes or [output_size]
        self.quant_method.create_weights(self, input_size, self._local_rows(), self.params_dtype, self.device_)

    def _local_rows(self) -> int:
        return self.output_size_per_partition

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, shard_id=None) -> None:
        rows = param.shape[0]
        param.data.copy_(loaded_weight.narrow(0, self.tp_rank * rows, rows))

    def forward(self, x):
        y = self.quant_method.apply(self, x, self.bias)
        if self.gather_output and self.tp_size > 1:
            y = tensor_model_parallel_all_gather(y)
        return y, None


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel matrices fused along the output dimension (e.g. gate and up projections)."""

    def __init__(self, input_size, output_sizes: List[int], **kw):
        assert all(o % kw.get("tp_size", 1) == 0 for o in output_sizes)
        super().__init__(input_size, sum(output_sizes), output_sizes=list(output_sizes), **kw)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, shard_id: Optional[int] = None) -> None:
        if shard_id is None:
            # a checkpoint that already stores the fused matrix: split it into its logical parts first
            off = 0
            for i, size in enumerate(self.output_sizes):
                self.weight_loader(param, loaded_weight.narrow(0, off, size), i)
                off += size
            return
        size = self.output_sizes[shard_id] // self.tp_size
        dst_off = sum(self.output_sizes[:shard_id]) // self.tp_size
        param.data.narrow(0, dst_off, size).copy_(loaded_weight.narrow(0, self.tp_rank * size, size))


class QKVParallelLinear(ColumnParallelLinear):
    """Fused q | k | v projection; rank r holds its q heads and its (possibly replicated) kv heads."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int, total_num_kv_heads: Optional[int] = None,
                 bias: bool = False, tp_size: int = 1, tp_rank: int = 0, params_dtype=None, device="cpu", prefix=""):
        self.hidden_size, self.head_size = hidden_size, head_size
        self.total_num_heads = total_num_heads
        self.total_num_kv_heads = total_num_kv_heads or total_num_heads
        self.num_heads = total_num_heads // tp_size
        if tp_size >= self.total_num_kv_heads:
            self.num_kv_heads, self.num_kv_head_replicas = 1, tp_size // self.total_num_kv_heads
        else:
            self.num_kv_heads, self.num_kv_head_replicas = self.total_num_kv_heads // tp_size, 1
        out = (self.num_heads + 2 * self.num_kv_heads) * tp_size * head_size
        LinearBase.__init__(self, hidden_size, out, params_dtype, device, prefix)
        self.tp_size, self.tp_rank, self.gather_output = tp_size, tp_rank, False
        self.output_sizes = [self.num_heads * head_size * tp_size, self.num_kv_heads * head_size * tp_size,
                             self.num_kv_heads * head_size * tp_size]
        self.output_size_per_partition = (self.num_heads + 2 * self.num_kv_heads) * head_size
        self.quant_method.create_weights(self, hidden_size, self.output_size_per_partition, self.params_dtype, self.device_)

    def _shard(self, shard_id: str) -> Tuple[int, int]:
        hs = self.head_size
        return {"q": (0, self.num_heads * hs), "k": (self.num_heads * hs, self.num_kv_heads * hs),
                "v": ((self.num_heads + self.num_kv_heads) * hs, self.num_kv_heads * hs)}[shard_id]

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, shard_id: Optional[str] = None) -> None:
        if shard_id is None:
            # fused checkpoint tensor [q | k | v] over all heads
            hs = self.head_size
            q_rows, kv_rows = self.total_num_heads * hs, self.total_num_kv_heads * hs
            self.weight_loader(param, loaded_weight.narrow(0, 0, q_rows), "q")
            self.weight_loader(param, loaded_weight.narrow(0, q_rows, kv_rows), "k")
            self.weight_loader(param, loaded_weight.narrow(0, q_rows + kv_rows, kv_rows), "v")
            return
        off, size = self._shard(shard_id)
        src_rank = self.tp_rank if shard_id == "q" else self.tp_rank // self.num_kv_head_replicas
        param.data.narrow(0, off, size).copy_(loaded_weight.narrow(0, src_rank * size, size))


class RowParallelLinear(LinearBase):
    """Y = X A^T with A split along its input columns; partial results are summed over the TP group."""

    def __init__(self, input_size, output_size, bias: bool = False, input_is_parallel: bool = True,
                 reduce_results: bool = True, tp_size: int = 1, tp_rank: int = 0, params_dtype=None, device="cpu", prefix=""):
        super().__init__(input_size, output_size, params_dtype, device, prefix)
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.input_is_parallel, self.reduce_results = input_is_parallel, reduce_results
        assert input_size % tp_size == 0
        self.input_size_per_partition = input_size // tp_size
        self.quant_method.create_weights(self, self.input_size_per_partition, output_size, self.params_dtype, self.device_)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, shard_id=None) -> None:
        cols = param.shape[1]
        param.data.copy_(loaded_weight.narrow(1, self.tp_rank * cols, cols))

    def forward(self, x):
        if not self.input_is_parallel and self.tp_size > 1:
            x = x.narrow(-1, self.tp_rank * self.input_size_per_partition, self.input_size_per_partition).contiguous()
        y = self.quant_method.apply(self, x, None)
        if self.reduce_results and self.tp_size > 1:
            y = tensor_model_parallel_all_reduce(y)
        return y, None
