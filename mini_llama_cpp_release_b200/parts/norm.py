"""RMSNorm, fused with the residual addition that precedes it.

y_i = x_i · 1/sqrt(mean(x²) + eps) · w_i: eps inside the square root, multiply order
x·scale·w, statistics in float32 (src/ops.cpp:19-41).  The reference adds a branch's
output to the residual stream with a separate pass (src/forward.cpp:772, 779); here that
addition rides in the next norm's kernel, in float32, and the stream itself stays float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part, TensorSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    graph_safe = True

    def __init__(self, name: str, size: int, eps: float):
        super().__init__(name, size=size, eps=eps)
        self.size = int(size)
        self.eps = float(eps)

    def tensors(self):
        return [TensorSpec(self.name + "weight", (self.size,), role="gain", init="one_plus_normal")]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.gain = get(self.name + "weight").to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.gain.numel() * 4

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x: float32 [n, size], updated in place to x + delta when delta is given."""
        out = self.runtime.empty(*x.shape, dtype=out_dtype or self.runtime.dtype)
        kernels.add_rmsnorm(x, delta, self.gain, self.eps, out)
        return out
