"""y = x · Wᵀ for a weight stored [out, in] (src/matmul_optimized.cpp:40-54), the one
contraction every part is made of.

Which kernel runs is decided by the operand types, never by the model:
  * any float32 operand (the whole 32-bit path, or a tensor the checkpoint stores in
    32-bit while the engine computes in bfloat16): the float32 multiply-add kernel of
    csrc/linear_simt.cu.  No tensor-core mode takes part.
  * bfloat16 × bfloat16: the tensor-core matrix product with float32 accumulation.  Where
    the reference calls cuBLAS for its linears (src/cuda_matmul.cpp:216-233) the library
    product stands here too.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, runtime: Runtime):
        assert weight.dim() == 2
        self.weight = weight.contiguous()
        self.runtime = runtime
        self.out_features, self.in_features = weight.shape

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype = torch.float32,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert x.dim() == 2 and x.shape[1] == self.in_features, (x.shape, self.weight.shape)
        m = x.shape[0]
        if out is None:
            out = self.runtime.empty(m, self.out_features, dtype=out_dtype)
        if x.dtype == torch.float32 or self.weight.dtype == torch.float32:
            kernels.linear_simt(x, self.weight, out)
            return out
        kernels.require_cuda(x)
        if out.dtype == torch.float32:
            torch.mm(x, self.weight.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, self.weight.t(), out=out)
        kernels.count_library_launches(1)
        return out
