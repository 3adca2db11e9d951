"""y = x · Wᵀ for a weight stored [out, in] (src/matmul_optimized.cpp:40-54), the one
contraction every part is made of.

Which kernel runs is decided by the operand types and sizes, never by the model:
  * any float32 operand (the whole 32-bit path, or a tensor the checkpoint stores in
    32-bit while the engine computes in bfloat16): the float32 multiply-add kernel of
    csrc/linear_simt.cu.  No tensor-core mode takes part.
  * bfloat16 × bfloat16 with an inner size that is a multiple of 8: the tcgen05/TMA kernel of
    csrc/gemm_tcgen05.cu, always when an epilogue is fused (Q/K/V with bias, rotation and
    cache write; gate/up with SiLU·mul), and for plain products of up to 64 rows (decoding),
    where the K range is split over blocks and the partial sums are left to the consumer.
  * plain bfloat16 products of more rows (prompts): the tokens-as-M tcgen05 kernels, one SM
    per tile (csrc/gemm_tcgen05_rows.cu) or, when tiles of 256 x 256 fill the GPU twice
    over, a pair of SMs per tile (csrc/gemm_tcgen05_pair.cu); where the product is a
    branch's last it adds into the float32 residual stream in its epilogue, with the K range
    shared out over blocks when the tiles alone would leave SMs idle.
  * bfloat16 products whose sizes those kernels do not take (an inner size that is no
    multiple of 8; in a prompt, a row count of W that is no multiple of 16): the library's
    product with float32 accumulation, as the reference calls cuBLAS for all of its linears
    (src/cuda_matmul.cpp:216-233).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Runtime

SMALL_BATCH = 64          # up to this many rows a plain product runs on the tcgen05 kernel with split K
MAX_SPLITS = 8            # partial sums the consumer has to add
ADD_MAX_SPLITS = 24       # splits of a product that adds into the stream atomically (nobody has to add them up)
ADD_MAX_SPLITS_SOME = 10  # the same for 2 to 16 rows


def add_split_cap(n_tok: int) -> int:
    """The most blocks that share the K range of a few-row product that adds into the stream.  More blocks stream the
    weights faster, but every block adds its part with one atomic per row and column, and its blocks are SMs on which
    the kernel after it cannot start early to ask for its own weights.  Measured on whole decode steps of 24 and 28
    layers on a B200, caps of 8 / 10 / 12 / 24: 0.733 / 0.710 / 0.717 / 0.722 ms at 8 rows and 1.271 against 1.300 ms
    (10 against 24) at 16 rows of the Qwen2-1.5B sizes, but 0.735 / 0.703 / 0.704 / 0.683 ms at one row and
    1.039 / 1.044 / 1.016 / 1.009 ms at 64 rows; at the 7B sizes the cap does not bind."""
    return ADD_MAX_SPLITS_SOME if 2 <= n_tok <= 16 else ADD_MAX_SPLITS


def split_count(n_out: int, k: int, n_tok: int, n_sms: int, max_splits: int = 0) -> int:
    """How many blocks share the K range of a skinny product: enough to occupy the SMs, each
    with at least two 64-element K steps."""
    if n_tok > SMALL_BATCH:
        return 1
    row_tiles = (n_out + 127) // 128
    k_blocks = (k + 63) // 64
    s = max(1, min(n_sms // max(1, row_tiles), k_blocks // 2, max_splits or MAX_SPLITS))
    per = (k_blocks + s - 1) // s
    return (k_blocks + per - 1) // per


class Linear:
    def __init__(self, weight: torch.Tensor, runtime: Runtime):
        assert weight.dim() == 2
        self.weight = weight.contiguous()
        self.runtime = runtime
        self.out_features, self.in_features = weight.shape
        self.tensor_core_ok = (weight.dtype == torch.bfloat16 and self.in_features % 8 == 0
                               and self.weight.data_ptr() % 16 == 0)

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def can_add_into_stream(self, n_rows: int) -> bool:
        """Whether `add_into` has a kernel for these operands: the tcgen05 products (atomic adds for few rows; plain or
        atomic adds for more), else the library's product with the stream as the matrix it adds to."""
        return self.tensor_core_ok

    def add_into(self, x: torch.Tensor, stream: torch.Tensor) -> None:
        """stream (float32 [n, out]) += x · Wᵀ.  Few rows: the weights-as-M tcgen05 product, the K range shared out over
        as many blocks as is useful.  More rows: the tokens-as-M tcgen05 product, with a K split when its tiles alone
        would leave SMs idle (the library's product only for a row count that kernel does not take: no multiple of
        16).  Either way the stream is updated in the product's epilogue, so the norm that follows has one tensor to
        read, not two."""
        m = x.shape[0]
        if m > SMALL_BATCH and kernels.gemm_rows_takes(m, self.out_features, self.in_features):
            kernels.gemm_prompt(x, self.weight, stream, kernels.bindings.EPI_ADD, n_sms=self.runtime.n_sms)
            return
        if m > SMALL_BATCH:
            kernels.library_gemm(x, self.weight, stream, accumulate=True)
            return
        splits = split_count(self.out_features, self.in_features, m, self.runtime.n_sms, max_splits=add_split_cap(m))
        kernels.gemm_tcgen05(x, self.weight, stream, kernels.bindings.EPI_ADD, splits, n_sms=self.runtime.n_sms)

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype = torch.float32, partial_ok: bool = False) -> torch.Tensor:
        """[n, out] in `out_dtype`; with `partial_ok` possibly float32 partial sums [slices, n, out]
        whose sum over the first axis is the product."""
        assert x.dim() == 2 and x.shape[1] == self.in_features, (x.shape, self.weight.shape)
        rt = self.runtime
        m = x.shape[0]
        if x.dtype == torch.float32 or self.weight.dtype == torch.float32:
            out = rt.empty(m, self.out_features, dtype=out_dtype)
            kernels.linear_simt(x, self.weight, out)
            return out
        kernels.require_cuda(x)
        if self.tensor_core_ok and m <= SMALL_BATCH:
            splits = split_count(self.out_features, self.in_features, m, rt.n_sms) if (partial_ok and out_dtype == torch.float32) else 1
            out = rt.empty(splits, m, self.out_features, dtype=out_dtype)
            kernels.gemm_tcgen05(x, self.weight, out, kernels.bindings.EPI_STORE, splits, n_sms=rt.n_sms)
            return out if splits > 1 else out[0]
        out = rt.empty(m, self.out_features, dtype=out_dtype)
        if self.tensor_core_ok and kernels.gemm_rows_takes(m, self.out_features, self.in_features):
            kernels.gemm_prompt(x, self.weight, out, kernels.bindings.EPI_STORE, n_sms=rt.n_sms)
        else:
            kernels.library_gemm(x, self.weight, out)
        return out
