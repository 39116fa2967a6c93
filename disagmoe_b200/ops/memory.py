"""Token permutation helpers (reference: disagmoe/ops/memory.py:33-101).

``get_mappings_from_exp_ids`` is the counting sort that turns per-row expert ids into destination rows;
``permute_tokens_cuda`` / ``permute_tokens`` run the row scatter on the device kernel
(``csrc/kernels/elementwise.cu: permute_rows_kernel``; any hidden size that is a multiple of 8, 16-byte accesses).
"""
from __future__ import annotations

from typing import List, Tuple, Union

import torch

from . import functional as F


def get_mappings_from_exp_ids(exp_ids: Union[torch.Tensor, List[int]], num_experts: int) -> Tuple[List[int], List[int]]:
    """Stable counting sort: returns (mappings, counts) with ``sorted[mappings[i]] = tokens[i]``."""
    if isinstance(exp_ids, torch.Tensor):
        exp_ids = exp_ids.view(-1).tolist()
    counts = [0] * num_experts
    for e in exp_ids:
        counts[e] += 1
    start, run = [0] * num_experts, 0
    for e in range(num_experts):
        start[e] = run
        run += counts[e]
    mappings = [0] * len(exp_ids)
    for i, e in enumerate(exp_ids):
        mappings[i] = start[e]
        start[e] += 1
    return mappings, counts


def get_mappings_from_exp_ids_cuda(exp_ids: torch.Tensor, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same result computed on the device (no host round trip)."""
    flat = exp_ids.view(-1).long()
    order = torch.sort(flat, stable=True).indices
    mappings = torch.empty_like(order)
    mappings[order] = torch.arange(flat.numel(), device=flat.device)
    counts = torch.bincount(flat, minlength=num_experts)
    return mappings.int(), counts


def permute_tokens_cuda(tokens: torch.Tensor, mappings: torch.Tensor) -> torch.Tensor:
    """out[mappings[i]] = tokens[i // k] with k = len(mappings) / len(tokens) (k > 1 duplicates rows for top-k)."""
    n_out = mappings.numel()
    repeat = max(1, n_out // max(1, tokens.shape[0]))
    return F.permute_rows(tokens, mappings.to(torch.int32), repeat=repeat, n_out=n_out)


permute_tokens = permute_tokens_cuda
# The reference also ships a Triton version of the same scatter (ops/memory.py:71-91, used by its tests only). This
# code base has no Triton path: the name resolves to the sm_100a kernel.
permute_tokens_triton = permute_tokens_cuda
