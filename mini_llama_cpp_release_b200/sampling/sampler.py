"""Choosing the next token: greedy, temperature, top-k.

Options and their meanings are the reference's (include/mini_llama/sampler.h:9-13;
src/sampler.cpp:92-152):
  temperature  float >= 0; below 1e-6 the choice is greedy; else weights exp((l - max)/T);
  top_k        int >= 0; 0 is off; 1 is greedy; k > 1 keeps the k largest logits (ties: lower
               id first), clamped to the vocabulary;
  seed         0 means "not reproducible" (a fresh seed per sampler), as in the reference.
`DeviceSampler` runs on the GPU and is what generation uses.  `HostSampler` is the same
procedure on host lists, for the generation loop's CPU tests and as a cross-check.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .rng import uniform_of

GREEDY_TEMPERATURE = 1e-6          # src/sampler.cpp:13


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 0

    def validate(self) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise ValueError("sampler: temperature must be finite and non-negative")       # src/sampler.cpp:26-30
        if self.top_k < 0:
            raise ValueError("sampler: top_k must be non-negative")                        # src/sampler.cpp:32-36

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_TEMPERATURE or self.top_k == 1                    # src/sampler.cpp:145-147

    def resolved_seed(self) -> int:
        return self.seed if self.seed != 0 else int.from_bytes(os.urandom(8), "little") | 1


class HostSampler:
    def __init__(self, params: SamplingParams):
        params.validate()
        self.params = params
        self.seed = params.resolved_seed()

    def sample(self, logits, seq_ids: Sequence[int], positions: Sequence[int]) -> List[int]:
        rows = logits.tolist() if hasattr(logits, "tolist") else [list(r) for r in logits]
        return [self._one(row, sid, pos) for row, sid, pos in zip(rows, seq_ids, positions)]

    def _one(self, row: List[float], seq_id: int, position: int) -> int:
        if not row:
            raise ValueError("sampler: cannot sample from empty logits")                  # src/sampler.cpp:16-18
        if any(not math.isfinite(v) for v in row):
            raise ValueError("sampler: logits must be finite")                            # src/sampler.cpp:19-23
        p = self.params
        if p.greedy:
            best = 0
            for i in range(1, len(row)):
                if row[i] > row[best]:
                    best = i
            return best
        ids = list(range(len(row)))
        if p.top_k > 1:
            ids.sort(key=lambda i: (-row[i], i))
            ids = ids[: min(p.top_k, len(row))]
        f32 = torch.float32
        v = torch.tensor([row[i] for i in ids], dtype=f32)
        w = torch.exp((v - v.max()) / torch.tensor(p.temperature, dtype=f32))
        target = torch.tensor(uniform_of(self.seed, seq_id, position), dtype=f32) * w.sum(dtype=f32)
        cum = torch.cumsum(w, dim=0)
        hit = torch.nonzero(cum >= target)
        return ids[int(hit[0])] if hit.numel() else ids[-1]


class DeviceSampler:
    """The sampler generation uses; `logits` is a float32 CUDA tensor [rows, vocab]."""

    def __init__(self, params: SamplingParams, device: torch.device):
        from .. import kernels
        params.validate()
        self.kernels = kernels
        self.params = params
        self.seed = params.resolved_seed()
        self.device = device

    def sample_device(self, logits: torch.Tensor, seq_ids: torch.Tensor, positions: torch.Tensor,
                      out: Optional[torch.Tensor] = None, seed_on_device: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 ids [rows] on the device; seq_ids and positions are int32 device tensors.  `seed_on_device`
        (two int32: the seed's halves), if given, is read by the kernel in place of this sampler's seed."""
        if out is None:
            out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        p = self.params
        if p.greedy:
            self.kernels.argmax(logits, out)
        else:
            self.kernels.sample(logits, p.temperature, p.top_k, self.seed, seq_ids, positions, out, seed_on_device)
        return out

    def sample(self, logits: torch.Tensor, seq_ids: Sequence[int], positions: Sequence[int]) -> List[int]:
        meta = torch.tensor([list(seq_ids), list(positions)], dtype=torch.int32).to(logits.device, non_blocking=True)
        return self.sample_device(logits, meta[0], meta[1]).tolist()
