"""Model placement: which device runs which attention layers and which (layer, expert) pairs, and the directed
edges tokens travel along (tokenizer -> layer-0 attention -> experts -> next attention ... -> sampler).

API and semantics follow the reference (disagmoe/utils/placement.py:29-537): ``ModelPlacement`` with its query
methods, ``ClusterConfig``, the strategies ``single`` / ``interleave`` / ``pipeline`` / ``colocate`` and
``get_model_placement``. The implementation is organised differently: every strategy only produces the two
tables (attention layers per device, experts per device, TP groups); edges, expert ranks and DP ranks are derived
from the tables by one shared routine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from itertools import count
from typing import Dict, List, Optional, Tuple

from ..config import ModelConfig
from .constants import GiB, SAMPLER_DEV_ID, TOKENIZER_DEV_ID


@dataclass
class ParallelConfig:
    tp: int = 1
    ep: int = 1
    dp: int = 1
    n_exp_per_rank: int = 1
    expert_ranks: Optional[Dict[Tuple[int, int], int]] = None

    @staticmethod
    def from_c(tp: int, ep: int, dp: int, n_exp_per_rank: int, expert_ranks: List):
        """Builds the native ParallelConfig (expert_ranks as a list of (layer, expert, rank) triples)."""
        from .. import disagmoe_c
        cfg = disagmoe_c.ParallelConfig()
        cfg.tp, cfg.ep, cfg.dp, cfg.n_exp_per_rank = tp, ep, dp, n_exp_per_rank
        cfg.expert_ranks = [tuple(x) for x in expert_ranks]
        return cfg


@dataclass
class ModelPlacement:
    attn: Dict[int, List[int]]                       # device -> attention layer ids
    expert: Dict[int, List[Tuple[int, int]]]         # device -> (layer id, expert id)
    tokenizer: int
    sampler: int
    in_device_ids: Dict[int, List[int]] = field(default_factory=dict)
    out_device_ids: Dict[int, List[int]] = field(default_factory=dict)
    device_groups: Optional[Dict[int, List[int]]] = None   # device -> its TP group (driver first)
    expert_ranks: Optional[Dict[Tuple[int, int], int]] = None
    attn_dp_ranks: Optional[Dict[int, int]] = None
    is_hybrid: bool = False

    # ---- queries -------------------------------------------------------------------------------------------
    def expert_rank_at(self, device_id: int, num_expert_per_rank: int = 0) -> int:
        ranks = {self.expert_ranks[pair] for pair in self.expert[device_id]}
        assert len(ranks) == 1, f"device {device_id} holds experts of several EP ranks: {ranks}"
        return ranks.pop()

    def attn_rank_at(self, device_id: int) -> int:
        assert device_id in self.attn
        group = (self.device_groups or {}).get(device_id, [device_id])
        return group.index(device_id) if device_id in group else 0

    def rank_at(self, device_id: int, *args, **kwargs) -> int:
        if device_id in self.expert and self.expert[device_id]:
            return self.expert_rank_at(device_id, *args, **kwargs)
        return self.attn_rank_at(device_id)

    def out_expert_ranks_at(self, device_id: int) -> List[Tuple[int, int, int]]:
        out = []
        for dst in self.out_device_ids.get(device_id, []):
            for layer_id, expert_id in self.expert.get(dst, []):
                out.append((layer_id, expert_id, self.expert_ranks[(layer_id, expert_id)]))
        return out

    def attn_layer_ids_at(self, device_id: int) -> List[int]:
        return self.attn.get(device_id, [])

    def expert_ids_at(self, device_id: int) -> List[Tuple[int, int]]:
        return self.expert.get(device_id, [])

    def attn_dp_rank_at(self, device_id: int) -> int:
        return (self.attn_dp_ranks or {}).get(device_id, 0)

    def layer_ids_at(self, device_id: int) -> List[int]:
        layers = set(self.attn.get(device_id, [])) | {l for l, _ in self.expert.get(device_id, [])}
        return sorted(layers)

    def add_edge(self, start: int, end: int) -> None:
        ins = self.in_device_ids.setdefault(end, [])
        outs = self.out_device_ids.setdefault(start, [])
        if start not in ins:
            ins.append(start)
            outs.append(end)

    def is_worker_device(self, device_id: int) -> bool:
        """True for the non-driver members of a TP group."""
        g = (self.device_groups or {}).get(device_id)
        return g is not None and g[0] != device_id

    def has_attn(self, device_id: int) -> bool:
        return device_id in self.attn and len(self.attn[device_id]) > 0

    def has_expert(self, device_id: int) -> bool:
        return device_id in self.expert and len(self.expert[device_id]) > 0

    def in_device_ids_at(self, device_id: int, tp_enable_inter_group: bool) -> List[int]:
        if self.is_worker_device(device_id) and tp_enable_inter_group:
            driver = self.device_groups[device_id][0]
            return [d for d in self.in_device_ids.get(driver, []) if d not in (self.tokenizer, self.sampler)]
        return self.in_device_ids.get(device_id, [])

    def device_ids(self) -> List[int]:
        return sorted(set(self.attn) | set(self.expert))

    def attn_devices_of_layer(self, layer_id: int) -> List[int]:
        return sorted(d for d, ls in self.attn.items() if layer_id in ls)

    def expert_devices_of_layer(self, layer_id: int) -> List[int]:
        return sorted(d for d, pairs in self.expert.items() if any(l == layer_id for l, _ in pairs))


@dataclass
class ClusterConfig:
    n_node: int
    n_gpu: int
    gpu_cap: float = 180 * GiB          # B200: 180 GB HBM3e per GPU
    id_tokenizer: int = TOKENIZER_DEV_ID
    id_sampler: int = SAMPLER_DEV_ID


class PlacementBase:
    def __init__(self, model_config: ModelConfig, cluster_config: ClusterConfig, step_attn: int = 0,
                 step_expert: int = 0, zigzag_attn: bool = True):
        self.model_config = model_config
        self.cluster_config = cluster_config

    tp_size = property(lambda self: self.model_config.tp_size)
    ep_size = property(lambda self: self.model_config.ep_size)
    dp_size = property(lambda self: self.model_config.dp_size)
    num_layers = property(lambda self: self.model_config.num_layers)

    # strategy hook: returns a ModelPlacement with attn / expert / device_groups filled in
    def _solve(self, n_layer: int, n_expert: int, n_node: int, n_gpu_per_node: int) -> ModelPlacement:
        raise NotImplementedError

    def _add_edges(self, place: ModelPlacement) -> ModelPlacement:
        L = self.num_layers
        attn_of = {l: place.attn_devices_of_layer(l) for l in range(L)}
        exp_of = {l: place.expert_devices_of_layer(l) for l in range(L)}
        for l in range(L):
            if l == 0:
                for d in attn_of[0]:
                    place.add_edge(place.tokenizer, d)
                for d in attn_of[0]:
                    # with TP only the driver of a group talks to the sampler
                    if self.tp_size > 1 and place.is_worker_device(d):
                        continue
                    place.add_edge(place.sampler, d)
            else:
                for d in attn_of[l]:
                    for prev in exp_of[l - 1]:
                        place.add_edge(prev, d)
            if l == L - 1:
                for d in exp_of[l]:
                    place.add_edge(d, place.sampler)
            for d in attn_of[l]:
                for e in exp_of[l]:
                    place.add_edge(d, e)
        return place

    def _update_expert_rank(self, place: ModelPlacement) -> ModelPlacement:
        per = self.model_config.num_experts_per_rank
        place.expert_ranks = {(l, e): e // per for l in range(self.num_layers)
                              for e in range(self.model_config.num_experts)}
        return place

    def _update_attn_dp_rank(self, place: ModelPlacement) -> ModelPlacement:
        place.attn_dp_ranks = {d: 0 for d in place.attn}
        return place

    def solve(self) -> ModelPlacement:
        place = self._solve(self.num_layers, self.model_config.num_experts, self.cluster_config.n_node,
                            self.cluster_config.n_gpu)
        place.tokenizer = self.cluster_config.id_tokenizer
        place.sampler = self.cluster_config.id_sampler
        place = self._add_edges(place)
        place = self._update_expert_rank(place)
        place = self._update_attn_dp_rank(place)
        return place


class SinglePlacement(PlacementBase):
    """One device per attention replica and one per expert, for every layer (layers x (rep_attn + experts) GPUs)."""

    def __init__(self, model_config, cluster_config, rep_attn: int = 1):
        super().__init__(model_config, cluster_config)
        self.rep_attn = rep_attn

    def _solve(self, n_layer, n_expert, n_node, n_gpu_per_node):
        assert n_layer * (self.rep_attn + n_expert) <= n_node * n_gpu_per_node, "not enough devices"
        ids = count()
        attn, expert = {}, {}
        for l in range(n_layer):
            for _ in range(self.rep_attn):
                attn[next(ids)] = [l]
            for e in range(n_expert):
                expert[next(ids)] = [(l, e)]
        groups = {d: [d] for d in attn}
        return ModelPlacement(attn, expert, -1, -1, device_groups=groups)

    def _update_expert_rank(self, place):
        place.expert_ranks = {(l, e): e for l in range(self.num_layers) for e in range(self.model_config.num_experts)}
        return place


class InterleavePlacement(PlacementBase):
    """Devices are cut into groups of (tp attention + ep expert) GPUs; layer l runs on group l mod n_groups."""

    def _solve(self, n_layer, n_expert, n_node, n_gpu_per_node):
        tp, ep = self.tp_size, self.ep_size
        n_dev = n_node * n_gpu_per_node
        assert n_dev % (tp + ep) == 0, "devices must split into groups of tp + ep"
        n_group = n_dev // (tp + ep)
        per = self.model_config.num_experts_per_rank
        attn, expert, groups = {}, {}, {}
        for g in range(n_group):
            base = g * (tp + ep)
            tp_devs = list(range(base, base + tp))
            for d in tp_devs:
                attn[d] = [l for l in range(n_layer) if l % n_group == g]
                groups[d] = tp_devs
            for r in range(ep):
                d = base + tp + r
                expert[d] = [(l, e) for l in range(n_layer) if l % n_group == g
                             for e in range(r * per, (r + 1) * per)]
        return ModelPlacement(attn, expert, -1, -1, device_groups=groups)


class PipelinePlacement(PlacementBase):
    """Layers are striped over ``step_attn`` attention stages and ``step_expert`` expert stages.

    Attention stage i (layers l with l mod p == i when zigzag, else a contiguous range) is replicated dp times,
    each replica a TP group: devices [0, p * dp * tp). Expert stage j (layers l mod q == j) is an EP group of
    ep devices placed after all attention devices.
    """

    def __init__(self, model_config, cluster_config, step_attn: int, step_expert: int, zigzag_attn: bool = True):
        super().__init__(model_config, cluster_config)
        self.step_attn, self.step_expert, self.zigzag_attn = step_attn, step_expert, zigzag_attn

    def _stage_layers(self) -> Tuple[List[List[int]], List[List[int]]]:
        p, q, L = self.step_attn, self.step_expert, self.num_layers
        a = [[] for _ in range(p)]
        e = [[] for _ in range(q)]
        for l in range(L):
            a[l % p if self.zigzag_attn else min(p - 1, l // max(1, L // p))].append(l)
            e[l % q].append(l)
        return a, e

    def _solve(self, n_layer, n_expert, n_node, n_gpu_per_node):
        p, q, tp, dp, ep = self.step_attn, self.step_expert, self.tp_size, self.dp_size, self.ep_size
        n_attn = p * tp * dp
        need = n_attn + q * ep
        assert n_node * n_gpu_per_node >= need, f"placement needs {need} GPUs, {n_node * n_gpu_per_node} available"
        a_layers, e_layers = self._stage_layers()
        per = self.model_config.num_experts_per_rank
        attn = {d: [] for d in range(n_attn)}
        groups = {}
        for stage in range(p):
            for rep in range(dp):
                driver = (stage * dp + rep) * tp
                members = list(range(driver, driver + tp))
                for d in members:
                    groups[d] = members
                    # every member of a TP group computes its head shard of every layer of the stage
                    attn[d] = list(a_layers[stage])
        expert = {d: [] for d in range(n_attn, n_attn + q * ep)}
        for stage in range(q):
            for e in range(n_expert):
                d = n_attn + stage * ep + e // per
                expert[d].extend((l, e) for l in e_layers[stage])
        for d in expert:
            expert[d].sort()
        return ModelPlacement(attn, expert, -1, -1, device_groups=groups)

    def _update_attn_dp_rank(self, place):
        place.attn_dp_ranks = {d: (d // self.tp_size) % self.dp_size for d in place.attn}
        return place


class ColocatePlacement(PlacementBase):
    """Every device runs all attention layers (one DP replica each) and one EP shard of every layer's experts."""

    def _solve(self, n_layer, n_expert, n_node, n_gpu_per_node):
        n_dev = n_node * n_gpu_per_node
        per = self.model_config.num_experts_per_rank
        attn = {d: list(range(n_layer)) for d in range(n_dev)}
        expert = {d: [] for d in range(n_dev)}
        for l in range(n_layer):
            for e in range(n_expert):
                expert[e // per].append((l, e))
        return ModelPlacement(attn, expert, -1, -1, device_groups={d: [d] for d in range(n_dev)}, is_hybrid=True)

    def _update_attn_dp_rank(self, place):
        place.attn_dp_ranks = {d: d for d in place.attn}
        return place


_placement_cls = {
    "colocate": ColocatePlacement,
    "single": SinglePlacement,
    "interleave": InterleavePlacement,
    "pipeline": PipelinePlacement,
}


def get_model_placement(model_config: ModelConfig, cluster_config: ClusterConfig, strategy: str = "single",
                        *args, verbose: bool = False, **kwargs) -> ModelPlacement:
    if strategy not in _placement_cls:
        raise NotImplementedError(f"unknown placement strategy {strategy!r}")
    cls = _placement_cls[strategy]
    if strategy == "pipeline":
        solver = cls(model_config, cluster_config, *args, **kwargs)
    elif strategy == "single":
        solver = cls(model_config, cluster_config, *args, **kwargs)
    else:
        solver = cls(model_config, cluster_config)
    place = solver.solve()
    if verbose:
        print(f"Model Placement: {place}")
    return place
