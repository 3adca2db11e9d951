"""The arrangement of a layer's parts around the residual stream.

Pre-norm: x ← x + mixer(norm(x)); x ← x + feed_forward(norm(x)) (src/forward.cpp:726-780).
The additions are deferred: a branch's output travels as `pending` and is added, in
float32, by the next norm's kernel — the block's own second norm, the next block's first
norm, or the model's final norm.  On the tensor-core path of small steps the addition moves into
the preceding product's epilogue (atomic adds into the stream) and nothing is pending at all."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config.registry import register_part, build_part
from ..config.specs import PartSpec
from .base import MixerMemory, Part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    graph_safe = True

    def __init__(self, name: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec, names: Optional[dict] = None):
        super().__init__(name)
        names = names or {}
        self.mixer_norm = build_part(mixer_norm, name + names.get("mixer_norm", "mixer_norm."))
        self.mixer = build_part(mixer, name + names.get("mixer", "mixer."))
        self.feed_forward_norm = build_part(feed_forward_norm, name + names.get("feed_forward_norm", "feed_forward_norm."))
        self.feed_forward = build_part(feed_forward, name + names.get("feed_forward", "feed_forward."))

    def children(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], step, memory: MixerMemory
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """A part either adds its output into the stream x itself (`accumulates`, asked through `residual=x`;
        it then returns None) or returns its output, which waits in `pending` for the next norm to add it."""
        mixer, ffn = self.mixer, self.feed_forward
        h = self.mixer_norm.forward(x, pending)
        a = mixer.forward(h, step, memory, residual=x) if getattr(mixer, "accumulates", False) else mixer.forward(h, step, memory)
        h2 = self.feed_forward_norm.forward(x, a)
        f = ffn.forward(h2, step, residual=x) if getattr(ffn, "accumulates", False) else ffn.forward(h2, step)
        return x, f
