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
    """One layer: an arrangement (`block`) of a mixer and a feed-forward, each behind its
    norm.  `name` is the prefix of the layer's tensors in the checkpoint."""
    name: str
    block: str                      # kind of the arrangement, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    names: Mapping[str, str] = field(default_factory=dict)   # role → the part's prefix below `name`

    def block_spec(self) -> PartSpec:
        return PartSpec("block", self.block, dict(mixer=self.mixer, feed_forward=self.feed_forward,
                                                  mixer_norm=self.mixer_norm,
                                                  feed_forward_norm=self.feed_forward_norm, names=dict(self.names)))


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
