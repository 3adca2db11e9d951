"""Rotate-half ("neox") rotary position encoding.

For pair i of a head, f_i = 1 / theta^(2i/hd); the angle p·f_i is a float32 product of the
integer position and the float32 frequency; (x_i, x_{i+hd/2}) ← (x_i·c − x_{i+hd/2}·s,
x_i·s + x_{i+hd/2}·c) (src/ops.cpp:125-141).  The frequencies are computed on the host the
way the reference computes them; cos and sin are tabulated once per context on the device
and every kernel reads the table.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part


def neox_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """f_i as float32: the exponent 2i/hd is a float32 quotient, the power is rounded to
    float32, then 1/x in float32 (src/ops.cpp:132)."""
    i2 = np.arange(0, head_dim, 2, dtype=np.float32)
    expo = i2 / np.float32(head_dim)
    power = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
    return torch.from_numpy((np.float32(1.0) / power).astype(np.float32))


# One table per (head size, theta, positions, device), shared by every layer and every model that asks for it: the
# attention layers of a model all rotate alike, and a decode step that pulled a private copy per layer through the
# cache hierarchy would read the same numbers two dozen times.
_TABLES: Dict[Tuple[int, float, int, str], torch.Tensor] = {}


def shared_table(inv_freq: torch.Tensor, head_dim: int, theta: float, max_positions: int) -> torch.Tensor:
    key = (head_dim, float(theta), max_positions, str(inv_freq.device))
    table = _TABLES.get(key)
    if table is None:
        table = _TABLES[key] = kernels.rope_table(inv_freq, max_positions)
    return table


@register_part("position", "rope_neox")
class RopeNeox(Part):
    graph_safe = True

    # How the attention part applies a position encoding.  `fusable = True`: the encoding is a rotation of the pairs
    # (i, i + head_dim/2) by angles that depend on the position alone; it offers `table`, [positions][head_dim/2][2]
    # float32 cos and sin (or None for "no rotation"), and the Q/K/V kernel's epilogue applies it.  `fusable = False`:
    # anything else; the attention part then calls `rotate(x, positions)` on the float32 queries and keys itself.
    fusable = True

    def __init__(self, name: str, head_dim: int, theta: float, max_positions: int):
        super().__init__(name, head_dim=head_dim, theta=theta, max_positions=max_positions)
        if head_dim <= 0 or head_dim % 2:
            raise ValueError(f"rope: head_dim must be positive and even, got {head_dim}")      # src/ops.cpp:164-168
        if not math.isfinite(theta) or theta <= 0:
            raise ValueError("rope: theta must be finite and positive")                        # src/ops.cpp:151-153
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)
        self.table: Optional[torch.Tensor] = None

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.inv_freq = neox_inv_freq(self.head_dim, self.theta).to(runtime.device)

    def prepare(self, n_positions: int) -> None:
        """Make sure the table exists.  It is built once, for every position the model allows,
        and never replaced: captured graphs keep reading the same memory."""
        if self.table is None:
            self.table = shared_table(self.inv_freq, self.head_dim, self.theta, self.max_positions)

    def rotate(self, x: torch.Tensor, positions: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Rotate float32 x [n, heads, head_dim] by int32 positions [n]; on its own, outside attention."""
        n, heads, hd = x.shape
        assert hd == self.head_dim
        self.prepare(int(positions.max().item()) + 1)
        out = self.runtime.empty(n, heads, hd, dtype=out_dtype or self.runtime.dtype)
        zeros = torch.zeros(n, dtype=torch.int32, device=x.device)
        kernels.qkv_post(x.reshape(n, heads * hd).contiguous(), None, positions, zeros, self.table, heads, 0, hd, out, None)
        return out


@register_part("position", "none")
class NoPosition(Part):
    graph_safe = True

    fusable = True

    def __init__(self, name: str, **_):
        super().__init__(name)
        self.table = None

    def prepare(self, n_positions: int) -> None:
        pass
