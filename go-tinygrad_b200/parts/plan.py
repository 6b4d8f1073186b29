"""The plan of a model: what its layers are made of and the order they run in.

A plan is data.  An architecture's registry entry produces it from the typed
configuration; the engine builds parts from it and runs the schedule.  No part
knows which model it is in: a part sees only its own `PartSpec` (a kind, looked
up in the part registries, and its sizes and constants as parameters).

The reference does the opposite: one loop body with ``if ModelType == ...``
branches (model/llama.go:1094-1455) and per-layer flags such as ``HasKV`` and
``KVSourceLayer`` (model/llama.go:679-695, model/kv_staging.go:11-54) for layers
that reuse another layer's cache.  Those needs are expressed here as schedule
entries.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """`kind` names a registered part of its category; `params` are its sizes,
    constants, weight names and nested PartSpecs (e.g. a mixer's position
    encoding)."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (`block`).  What the arrangement is made of --
    its mixer, feed-forward, norms, scalars of its own -- are nested PartSpecs
    among the block's parameters, under the names that block kind declares;
    the block builds and owns them.  Every layer carries its own spec, so
    mixers and feed-forwards may differ from layer to layer."""
    block: PartSpec

    def part(self, name: str) -> PartSpec:
        """The nested spec the block holds under `name`."""
        return self.block.params[name]

    def replace(self, **parts: Any) -> "LayerSpec":
        """The same layer with some of the block's parameters replaced."""
        return LayerSpec(PartSpec(self.block.kind, dict(self.block.params, **parts)))


def pre_norm_layer(mixer_norm: PartSpec, mixer: PartSpec, feed_forward_norm: PartSpec,
                   feed_forward: PartSpec) -> LayerSpec:
    """x += mixer(norm(x)); x += feed_forward(norm(x)): the ``pre_norm`` block."""
    return LayerSpec(PartSpec("pre_norm", {"mixer_norm": mixer_norm, "mixer": mixer,
                                           "feed_forward_norm": feed_forward_norm,
                                           "feed_forward": feed_forward}))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache` is the index of the schedule entry whose
    cache storage this run uses: None means its own.  An entry that points at
    another entry reads that entry's keys and values and writes none
    (`writes_cache` is then False).  A layer may appear in several entries; each
    entry that writes has storage of its own."""
    layer: int
    cache: Optional[int] = None

    @property
    def writes_cache(self) -> bool:
        return self.cache is None


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_tokens: Tuple[int, ...] = ()
    max_position: Optional[int] = None

    def check(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}; "
                                 f"the plan has {len(self.layers)} layers")
            if e.cache is not None:
                if not 0 <= e.cache < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache}, "
                                     f"which does not run before it")
                if self.schedule[e.cache].cache is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache}, "
                                     f"which has no storage of its own")


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i) for i in range(n_layers))


def plan_weight_specs(plan: ModelPlan) -> List[Any]:
    """Every tensor the plan's parts declare, built without touching a device."""
    from .base import build_part, walk  # late import: base imports this module
    roots = [build_part("embedding", plan.embedding)]
    roots += [build_part("block", layer.block) for layer in plan.layers]
    roots += [build_part("norm", plan.final_norm), build_part("head", plan.head)]
    specs = []
    for root in roots:
        for part in walk(root):
            specs += part.weight_specs()
    return specs
