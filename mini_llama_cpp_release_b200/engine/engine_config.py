"""How a model is run, as opposed to what it is: the engine's own typed configuration.

The reference keeps a `BackendConfig` (kind, device, quantisation, threads) that its command
line fills and validates before anything is loaded (include/mini_llama/backend.h:7-29;
src/backend.cpp:8-79).  Here there is one backend and no quantisation; what remains to
choose is the precision, the device, and three sizes that bound memory: how many tokens
the cache holds, how many sequences may be live, and how many tokens one step may run.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}

PAGE_TOKENS = 64          # the cache's unit; `max_tokens` counts each sequence rounded up to it


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


@dataclass(frozen=True)
class EngineConfig:
    """dtype             bfloat16 (tensor-core kernels, bfloat16 weights, activations and cache) or float32 (everything
                         in true 32-bit);
    device               a CUDA device ("cuda:0"); there is no other kind;
    max_tokens           the most tokens live sequences hold at any time, each sequence's count rounded up to 64:
                         sizes the cache;
    max_seqs             the most sequences live at any time (slots); default: one per 64 tokens of `max_tokens`, at
                         most 4096;
    max_batch_tokens     the most tokens one step runs at once: bounds the step's scratch memory.  `forward_batch`
                         cuts a larger batch into several steps, sequence by sequence."""
    dtype: object = "bfloat16"
    device: str = "cuda:0"
    max_tokens: int = 8192
    max_seqs: Optional[int] = None
    max_batch_tokens: int = 16384

    def __post_init__(self):
        object.__setattr__(self, "dtype", parse_dtype(self.dtype))
        object.__setattr__(self, "device", str(self.device))
        self.validate()

    def validate(self) -> None:
        dev = torch.device(self.device)
        if dev.type != "cuda":
            raise ValueError(f"device must be a CUDA device, got {self.device!r}: this engine has no CPU path")    # src/backend.cpp:40-52
        for name in ("max_tokens", "max_batch_tokens"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, int) or v < 1:
                raise ValueError(f"{name} must be a positive integer, got {v!r}")
        if self.max_seqs is not None and (isinstance(self.max_seqs, bool) or not isinstance(self.max_seqs, int) or self.max_seqs < 1):
            raise ValueError(f"max_seqs must be a positive integer or None, got {self.max_seqs!r}")

    @property
    def slots(self) -> int:
        """Sequences that may be live at once."""
        pages = (self.max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS
        return min(self.max_seqs, pages) if self.max_seqs is not None else min(pages, 4096)

    @property
    def dtype_name(self) -> str:
        return "bfloat16" if self.dtype == torch.bfloat16 else "float32"
