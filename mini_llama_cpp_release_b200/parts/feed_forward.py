"""SwiGLU feed-forward: down( gate·sigmoid(gate)·up ), no biases
(src/forward.cpp:672-702; src/ops.cpp:94-107).  Gate and up are one matrix product over
[Wgate; Wup]; the activation and the product are one kernel."""
from __future__ import annotations

import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part, TensorSpec
from .linear import Linear


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    graph_safe = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        super().__init__(name, hidden_size=hidden_size, intermediate_size=intermediate_size, activation=activation)
        if activation != "silu":
            raise ValueError(f"feed-forward: only the silu activation is supported (src/ops.cpp:94-107), got {activation!r}")
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)

    def tensors(self):
        n = self.name
        return [
            TensorSpec(n + "gate_proj.weight", (self.inter, self.hidden)),
            TensorSpec(n + "up_proj.weight", (self.inter, self.hidden)),
            TensorSpec(n + "down_proj.weight", (self.hidden, self.inter)),
        ]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        n = self.name
        self.gate_up = Linear(torch.cat([get(n + "gate_proj.weight"), get(n + "up_proj.weight")], dim=0), runtime)
        self.down = Linear(get(n + "down_proj.weight"), runtime)

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    def forward(self, h: torch.Tensor, step=None) -> torch.Tensor:
        rt = self.runtime
        gu = self.gate_up(h, rt.dtype)
        a = rt.empty(h.shape[0], self.inter)
        kernels.silu_mul(gu, a)
        return self.down(a, torch.float32)
