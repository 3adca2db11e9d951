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
        gate, up = get(n + "gate_proj.weight"), get(n + "up_proj.weight")
        # The fused product (SiLU·mul inside the tcgen05 kernel's epilogue) wants gate_j and up_j on
        # neighbouring rows: g0, u0, g1, u1, ...  Otherwise the rows are [gate; up].
        self.fused = runtime.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 \
            and self.hidden % 8 == 0
        if self.fused:
            w = torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden)
        else:
            w = torch.cat([gate, up], dim=0)
        self.gate_up = Linear(w, runtime)
        self.down = Linear(get(n + "down_proj.weight"), runtime)

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    accumulates = True        # forward(..., residual=x) may add the branch into the float32 stream and return None

    def forward(self, h: torch.Tensor, step=None, residual=None):
        rt = self.runtime
        a = rt.empty(h.shape[0], self.inter)
        if self.fused and kernels.gemm_rows_takes(h.shape[0], 2 * self.inter, self.hidden):
            kernels.gemm_prompt(h, self.gate_up.weight, a, kernels.bindings.EPI_SILU_MUL, n_sms=rt.n_sms)    # prompts
        elif self.fused:
            kernels.gemm_tcgen05(h, self.gate_up.weight, a, kernels.bindings.EPI_SILU_MUL, n_sms=rt.n_sms)
        else:
            kernels.silu_mul(self.gate_up(h, rt.dtype), a, interleaved=self.fused)
        if residual is not None and self.down.can_add_into_stream(h.shape[0]):
            self.down.add_into(a, residual)
            return None
        return self.down(a, torch.float32, partial_ok=True)
