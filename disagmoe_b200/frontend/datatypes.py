"""Python mirrors of the native records (reference: disagmoe/frontend/datatypes.py:6-205)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Tuple

from ..utils.constants import CPS


@dataclass
class ChannelInfo:
    expert_ids: List[Tuple[int, int]]
    attn_layer_ids: List[int]
    attn_dp_rank: int = 0

    def is_sampler_channel(self) -> bool:
        return len(self.expert_ids) == 0 and len(self.attn_layer_ids) == 0

    def to_c(self):
        from .. import disagmoe_c as C
        return C.ChannelInfo([tuple(e) for e in self.expert_ids], list(self.attn_layer_ids), self.attn_dp_rank)


@dataclass
class TokenMetadata:
    req_id: int
    exp_id: int
    attn_dp_rank: int
    init_prefill_len: int


@dataclass
class Metadata:
    shape: List[int]
    dtype: str
    layer_id: int
    req_ids: List[int]
    exp_ids: List[int]
    attn_dp_ranks: List[int]
    init_prefill_lens: List[int]
    topk_weights: List[float] = field(default_factory=list)
    positions: List[int] = field(default_factory=list)

    def num_tokens(self) -> int:
        return self.shape[0]

    @staticmethod
    def from_c(m) -> "Metadata":
        return Metadata(list(m.shape), m.dtype, m.layer_id, list(m.req_ids), list(m.exp_ids), list(m.attn_dp_ranks),
                        list(m.init_prefill_lens), list(m.topk_weights), list(m.positions))

    def to_c(self):
        from .. import disagmoe_c as C
        m = C.Metadata(list(self.shape))
        m.dtype, m.layer_id = self.dtype, self.layer_id
        m.req_ids, m.exp_ids, m.attn_dp_ranks = self.req_ids, self.exp_ids, self.attn_dp_ranks
        m.init_prefill_lens, m.topk_weights, m.positions = self.init_prefill_lens, self.topk_weights, self.positions
        return m


@dataclass
class AttentionBatchMetadata:
    layer_id: int
    shape: List[int]
    dtype: str
    num_prefill_seqs: int
    num_prefill_tokens: int
    num_decode_tokens: int
    seq_ids: List[int]
    init_prefill_lens: List[int]
    expert_ids: List[int]
    topk_weights: List[float]
    attn_dp_ranks: List[int]
    positions: List[int] = field(default_factory=list)

    @staticmethod
    def from_c(m) -> "AttentionBatchMetadata":
        return AttentionBatchMetadata(m.layer_id, list(m.shape), m.dtype, m.num_prefill_seqs, m.num_prefill_tokens,
                                      m.num_decode_tokens, list(m.seq_ids), list(m.init_prefill_lens),
                                      list(m.expert_ids), list(m.topk_weights), list(m.attn_dp_ranks), list(m.positions))

    def to_c(self):
        from .. import disagmoe_c as C
        m = C.AttentionBatchMetadata()
        for k in ("layer_id", "shape", "dtype", "seq_ids", "init_prefill_lens", "expert_ids", "topk_weights",
                  "attn_dp_ranks", "positions"):
            setattr(m, k, getattr(self, k))
        m.recount()
        return m


@dataclass
class SloStat:
    req_id: int
    t_prefill: float          # seconds: arrival of the first generated token
    t_prefill_std: float
    t_decode: float           # seconds: completion
    t_tokens: List[float]

    @staticmethod
    def from_c(s) -> "SloStat":
        return SloStat(s.req_id, s.t_prefill / CPS, s.t_prefill_std / CPS, s.t_decode / CPS,
                       [t / CPS for t in s.t_tokens])


@dataclass
class SamplerStepInfo:
    num_tokens: int
    time_stamp: float

    @staticmethod
    def from_c(s) -> "SamplerStepInfo":
        return SamplerStepInfo(s.num_tokens, s.time_stamp / CPS)


@dataclass
class TraceContext:
    msg: str
    t_start: float
    t_dur: float
    track_id: int

    @staticmethod
    def from_c(t) -> "TraceContext":
        return TraceContext(t.msg, t.t_start, t.t_dur, t.track_id)
