"""Model / cache / sampling configuration and the model presets.

Field names follow the reference's dataclasses (disagmoe/config.py:8-67) so that scripts written against it keep
working; the extra fields describe what the reference mocks away (vocabulary, RoPE, shared experts, dense
layers) and what the Blackwell kernels need to know.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import List, Optional

import torch


@dataclass
class ModelConfig:
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    num_experts: int
    intermediate_size: int
    dtype: torch.dtype
    ep_size: int
    tp_size: int = 1
    dp_size: int = 1
    rank: int = 0
    layer_ids: Optional[List[int]] = None
    top_k: int = 1

    tp_enable_inter_group: bool = True
    enable_cuda_graph_attn: bool = False
    enable_cuda_graph_expert: bool = False
    enable_grouped_gemm: bool = True

    graph_stride: int = 8
    max_batch_size_attn: int = 160
    max_batch_size_expert: int = 512
    max_seq_len: int = 4096

    enable_trace: bool = False

    # ---- real-model fields (the reference serves a mocked model and has none of these) ----
    vocab_size: int = 32000
    head_dim: Optional[int] = None              # default hidden_size // num_heads
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    norm_topk_prob: bool = True                 # renormalise the top-k router weights (Mixtral: yes)
    num_shared_experts: int = 0                 # always-on experts (Qwen-MoE: 1, DeepSeek-V2-Lite: 2)
    shared_intermediate_size: int = 0           # total ffn width of the shared expert(s)
    shared_expert_gate: bool = False            # sigmoid gate on the shared expert output (Qwen-MoE)
    first_k_dense: int = 0                      # leading layers with a dense FFN instead of experts
    dense_intermediate_size: int = 0
    eos_token_id: int = 2
    init_std: float = 0.02
    seed: int = 0
    name: str = "custom"

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_heads

    @property
    def num_experts_per_rank(self) -> int:
        return self.num_experts // self.ep_size

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def is_dense_layer(self, layer_id: int) -> bool:
        return layer_id < self.first_k_dense

    def clone(self, **changes) -> "ModelConfig":
        return replace(self, **changes)


@dataclass
class CacheConfig:
    """Paged KV cache configuration (field names of vLLM's CacheConfig as used at disagmoe/config.py:41-61)."""
    block_size: int = 16
    gpu_memory_utilization: float = 0.8
    swap_space: float = 0
    cache_dtype: str = "auto"
    num_gpu_blocks_override: Optional[int] = None
    sliding_window: Optional[int] = None
    enable_prefix_caching: bool = False
    cpu_offload_gb: float = 0
    num_reserved_blocks: int = 0
    num_gpu_blocks: Optional[int] = None
    num_cpu_blocks: Optional[int] = None


@dataclass
class SamplingConfig:
    min_output_len: int
    max_output_len: int


mixtral_config = ModelConfig(
    hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8, num_experts=8, intermediate_size=14336,
    dtype=torch.bfloat16, ep_size=8, top_k=2, vocab_size=32000, rope_theta=1e6, name="mixtral-8x7b",
)

duo_expert_mixtral = ModelConfig(
    hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8, num_experts=2, intermediate_size=14336,
    dtype=torch.bfloat16, ep_size=2, vocab_size=32000, rope_theta=1e6, name="mixtral-duo",
)

# Qwen1.5-MoE-A2.7B shape: 60 routed experts (top-4, no renormalisation) + one sigmoid-gated shared expert.
qwen_moe_config = ModelConfig(
    hidden_size=2048, num_layers=24, num_heads=16, num_kv_heads=16, num_experts=60, intermediate_size=1408,
    dtype=torch.bfloat16, ep_size=6, dp_size=2, top_k=4, vocab_size=151936, head_dim=128, rope_theta=1e6,
    rms_norm_eps=1e-6, norm_topk_prob=False, num_shared_experts=1, shared_intermediate_size=5632,
    shared_expert_gate=True, name="qwen1.5-moe-a2.7b",
)

# DeepSeek-V2-Lite shape with standard attention in place of MLA: first layer dense, 64 experts top-6, 2 shared.
deepseek_v2_lite_config = ModelConfig(
    hidden_size=2048, num_layers=27, num_heads=16, num_kv_heads=16, num_experts=64, intermediate_size=1408,
    dtype=torch.bfloat16, ep_size=8, tp_size=1, top_k=6, vocab_size=102400, head_dim=128, rope_theta=1e4,
    rms_norm_eps=1e-6, norm_topk_prob=False, num_shared_experts=2, shared_intermediate_size=2 * 1408,
    first_k_dense=1, dense_intermediate_size=10944, name="deepseek-v2-lite",
)

# Tiny Mixtral-style model of the CPU / fp32 correctness configuration.
tiny_config = ModelConfig(
    hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=4, num_experts=8, intermediate_size=512,
    dtype=torch.float32, ep_size=1, top_k=2, vocab_size=1024, head_dim=64, rope_theta=1e4, name="tiny-moe",
)

PRESETS = {
    "mixtral": mixtral_config, "mixtral-8x7b": mixtral_config, "duo": duo_expert_mixtral,
    "qwen-moe": qwen_moe_config, "deepseek-v2-lite": deepseek_v2_lite_config, "tiny": tiny_config,
}


def get_preset(name: str, **changes) -> ModelConfig:
    return PRESETS[name].clone(**changes)
