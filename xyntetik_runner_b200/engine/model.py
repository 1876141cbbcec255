"""A model as data: parts, and the order in which layers run.

``ModelPlan`` is what an architecture's builder returns: an embedding, a list
of blocks, a *schedule*, a final norm and a head.  The schedule is a list too:
an entry names the block to run and where its keys and values live.  It may
name a block twice (run the same weights again, with a cache entry of its own)
or let an entry read the cache that an earlier entry wrote
(``cache_from``; the reference keeps such an owner map per layer,
src/model.h:323-328).  ``LoadedModel`` binds the tensors and sorts the
schedule's cache entries into groups of equal need.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..cache.pages import GroupSpec
from ..parts.base import Block, KVNeed, Norm, Runtime, StateNeed
from ..parts.embedding import Embedding, Head
from ..weights.loader import TensorSource, TensorSpec, load_tensors


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                         # index into ModelPlan.blocks
    cache_from: Optional[int] = None   # index of an earlier schedule entry whose keys/values this one reads


@dataclass
class ModelPlan:
    embedding: Embedding
    blocks: List[Block]
    schedule: List[ScheduleEntry]
    final_norm: Norm
    head: Head
    width: int
    vocab_size: int
    max_positions: int
    stop_ids: Tuple[int, ...] = ()
    bos_id: Optional[int] = None

    def parts(self):
        return [self.embedding] + list(self.blocks) + [self.final_norm, self.head]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for p in self.parts():
            for name, spec in p.tensors().items():
                if name in out and out[name] != spec:
                    raise ValueError(f"tensor '{name}' is declared twice with different shapes")
                out[name] = spec
        return out

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            if e.cache_from is not None:
                if not (0 <= e.cache_from < i) or self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {i}: cache_from must name an earlier entry that owns a cache")
                a = self.blocks[e.layer].mixer.kv_need()
                b = self.blocks[self.schedule[e.cache_from].layer].mixer.kv_need()
                if a is None or b is None or (a.kv_heads, a.head_dim) != (b.kv_heads, b.head_dim):
                    raise ValueError(f"schedule entry {i}: cannot read the cache of entry {e.cache_from} (geometry differs)")


@dataclass
class LayerRuntime:
    """Where one schedule entry keeps its keys/values and its per-request state."""
    entry: int
    group: int = -1               # cache group, -1: this mixer keeps no keys
    layer_in_group: int = -1
    writes_cache: bool = False
    state: Optional[torch.Tensor] = None   # [max_requests, *shape], or None


@dataclass
class CacheGroupLayout:
    spec: GroupSpec
    kv_heads: int
    head_dim: int
    n_layers: int = 0


class LoadedModel:
    """Plan + tensors on the device + the cache layout the schedule implies."""

    def __init__(self, plan: ModelPlan, source: TensorSource, rt: Runtime):
        plan.validate()
        self.plan, self.rt = plan, rt
        tensors = load_tensors(plan.tensor_specs(), source, rt.device)
        for p in plan.parts():
            p.bind(tensors, rt)
        del tensors
        self.groups: List[CacheGroupLayout] = []
        self.layers: List[LayerRuntime] = []
        self.state_needs: List[Tuple[int, StateNeed]] = []
        keys: Dict[Tuple[int, int, Optional[int]], int] = {}
        for i, e in enumerate(plan.schedule):
            mixer = plan.blocks[e.layer].mixer
            lay = LayerRuntime(entry=i)
            need: Optional[KVNeed] = mixer.kv_need()
            if need is not None:
                if e.cache_from is not None:
                    src = self.layers[e.cache_from]
                    lay.group, lay.layer_in_group, lay.writes_cache = src.group, src.layer_in_group, False
                else:
                    key = (need.kv_heads, need.head_dim, need.window)
                    if key not in keys:
                        keys[key] = len(self.groups)
                        name = "full" if need.window is None else f"window{need.window}"
                        self.groups.append(CacheGroupLayout(GroupSpec(f"{name}:{need.kv_heads}x{need.head_dim}", need.window),
                                                            need.kv_heads, need.head_dim))
                    g = keys[key]
                    lay.group, lay.layer_in_group, lay.writes_cache = g, self.groups[g].n_layers, True
                    self.groups[g].n_layers += 1
            sn = mixer.state_need()
            if sn is not None:
                self.state_needs.append((i, sn))
            self.layers.append(lay)

    def kv_bytes_per_token(self, elem_size: int) -> int:
        return sum(2 * g.kv_heads * g.head_dim * g.n_layers * elem_size for g in self.groups)

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads: every scheduled block once, the final norm and the head
        (the embedding table is read by row only)."""
        total = sum(self.plan.blocks[e.layer].weight_bytes() for e in self.plan.schedule)
        return total + self.plan.final_norm.weight_bytes() + self.plan.head.weight_bytes()
