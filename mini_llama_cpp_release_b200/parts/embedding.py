"""Token embedding (x = E[token, :], src/forward.cpp:496-503) and the output head
(logits = W_lm · h, no bias, src/forward.cpp:849-853).  A tied head reads the embedding's
tensor instead of a copy of it (the reference copies: src/gguf_loader.cpp:436-443)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part, TensorSpec
from .linear import Linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int):
        super().__init__(name, vocab_size=vocab_size, hidden_size=hidden_size)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)

    def tensors(self):
        return [TensorSpec(self.name + "weight", (self.vocab, self.hidden), role="table")]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.table = get(self.name + "weight").contiguous()

    def weight_bytes(self) -> int:
        return 0      # a step touches one row per token, not the table

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = self.runtime.empty(token_ids.numel(), self.hidden, dtype=torch.float32)
        kernels.embed(self.table, token_ids, x)
        return x


@register_part("head", "linear_head")
class LinearHead(Part):
    graph_safe = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None):
        super().__init__(name, vocab_size=vocab_size, hidden_size=hidden_size, tied_to=tied_to)
        self.vocab, self.hidden, self.tied_to = int(vocab_size), int(hidden_size), tied_to

    def tensors(self):
        if self.tied_to:
            return [TensorSpec(self.tied_to, (self.vocab, self.hidden), role="table", stored=False)]
        return [TensorSpec(self.name + "weight", (self.vocab, self.hidden))]

    def ignorable_tensors(self):
        return [self.name + "weight"] if self.tied_to else []

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.proj = Linear(get(self.tied_to or (self.name + "weight")), runtime)

    def weight_bytes(self) -> int:
        return self.proj.nbytes()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.proj(h, torch.float32)
