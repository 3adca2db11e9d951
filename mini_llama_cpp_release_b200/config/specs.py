"""What a model is made of, as data.

An architecture's builder turns a `ModelConfig` into a `ModelSpec`: which part stands
where, with which sizes and constants, layer by layer, and in which order the layers
run.  The engine builds parts from these specifications through the part registry and
never looks at the architecture's name again.

The reference hard-wires one arrangement (src/forward.cpp:726-780, 896-898); the
specification below states that arrangement as data so that another one is another
builder, not another engine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .model_config import ModelConfig


@dataclass(frozen=True)
class PartSpec:
    """One part: `category` and `kind` pick the class in the part registry; `params` are
    its constructor's keyword arguments (every size and constant it needs)."""
    category: str
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: `block`, a part of category "block" whose parameters hold its own children (part specifications,
    as many and of whatever kinds that arrangement needs) and whatever else it takes.  `name` is the prefix of the
    layer's tensors in the checkpoint."""
    name: str
    block: PartSpec

    def child(self, role: str) -> Optional[PartSpec]:
        """The block's child part of that role ("mixer", "feed_forward", ...), if it has one."""
        v = self.block.params.get(role)
        return v if isinstance(v, PartSpec) else None

    @property
    def mixer(self) -> Optional[PartSpec]:
        return self.child("mixer")

    @property
    def feed_forward(self) -> Optional[PartSpec]:
        return self.child("feed_forward")


def prenorm_layer(name: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec,
                  names: Optional[Mapping[str, str]] = None) -> LayerSpec:
    """A layer in the pre-norm arrangement (src/forward.cpp:726-780): norm, mixer, residual; norm, feed-forward,
    residual.  `names`: role → the part's prefix below `name` in the checkpoint."""
    return LayerSpec(name, PartSpec("block", "prenorm", dict(
        mixer=mixer, feed_forward=feed_forward, mixer_norm=mixer_norm, feed_forward_norm=feed_forward_norm,
        names=dict(names or {}))))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelSpec.layers` and may appear in several
    entries (the same weights run twice).  Each entry has a cache of its own unless
    `reads_cache_of` names an earlier entry of the schedule, whose keys and values it
    then reads instead of writing any."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    config: ModelConfig
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    names: Mapping[str, str] = field(default_factory=lambda: {
        "embedding": "model.embed_tokens.", "final_norm": "model.norm.", "head": "lm_head."})

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for i, layer in enumerate(self.layers):
            if not isinstance(layer.block, PartSpec) or layer.block.category != "block":
                raise ValueError(f"layer {i}: `block` must be a part specification of category \"block\"")
        if not self.schedule:
            raise ValueError("the schedule is empty")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, which does not run before it")
                if self.schedule[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, which has none of its own")


def sequential_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Layers 0..n-1 once each, in order (src/forward.cpp:896-898)."""
    return tuple(ScheduleEntry(layer=i) for i in range(n_layers))
