"""Architecture-independent description of a decoder: which parts, in which order.

An architecture's typed configuration (for instance ``Qwen3Config``) is turned
into a ``ModelPlan`` by its builder.  Everything below the plan (parts, cache
manager, step function) reads only the plan, never the architecture's own
configuration, so no part knows which model it is in.

A plan is plain data:

* ``PartSpec``      : a part's kind (a registry key) and its parameters.
* ``LayerPlan``     : the parts of one layer and the checkpoint-name prefixes
                      under which their tensors are stored.
* ``ScheduleEntry`` : one execution of a layer.  The schedule is a list; it may
                      name a layer twice, and an entry may read the cache slot
                      that another entry writes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence


@dataclass(frozen=True)
class PartSpec:
    """Kind of a part (key in the part registry) with the part's parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **more: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(more)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerPlan:
    """One layer: a block arrangement over a mixer, a feed-forward and norms.

    ``names`` maps each part role to the checkpoint prefix of its tensors, e.g.
    ``{"mixer": "model.layers.3.self_attn.", "mixer_norm":
    "model.layers.3.input_layernorm."}``.
    """
    block: PartSpec
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    names: Mapping[str, str]


@dataclass(frozen=True)
class ScheduleEntry:
    """Run layer ``layer`` using cache slot ``cache_slot``.

    ``writes_cache`` is False for an entry that only reads what an earlier
    entry of the same step wrote into that slot.
    """
    layer: int
    cache_slot: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: Sequence[LayerPlan]
    schedule: Sequence[ScheduleEntry]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    names: Mapping[str, str]

    def __post_init__(self) -> None:
        n = len(self.layers)
        writers: dict[int, int] = {}
        for pos, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < n:
                raise ValueError(f"schedule entry {pos} names layer {entry.layer}, model has {n}")
            if entry.writes_cache:
                if entry.cache_slot in writers:
                    raise ValueError(
                        f"cache slot {entry.cache_slot} is written by schedule entries "
                        f"{writers[entry.cache_slot]} and {pos}")
                writers[entry.cache_slot] = pos
        for pos, entry in enumerate(self.schedule):
            if not entry.writes_cache:
                w = writers.get(entry.cache_slot)
                if w is None or w > pos:
                    raise ValueError(
                        f"schedule entry {pos} reads cache slot {entry.cache_slot} "
                        f"before any entry has written it")

    @property
    def num_cache_slots(self) -> int:
        return 1 + max((e.cache_slot for e in self.schedule), default=-1)


def default_schedule(num_layers: int) -> list[ScheduleEntry]:
    """Every layer once, in order, each with a cache slot of its own."""
    return [ScheduleEntry(layer=i, cache_slot=i) for i in range(num_layers)]
