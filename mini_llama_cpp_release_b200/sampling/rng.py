"""The uniform numbers of sampling, as a function of (seed, sequence id, position).

The reference seeds one `std::mt19937` per sampler and draws from it in order
(src/sampler.cpp:81-90, 67-69), so what a sequence draws depends on what was drawn before
it.  Here each draw is a hash of the seed, the sequence's id within the `generate` call and
the position of the token being chosen, so a sequence gets the same numbers alone, in a
batch, or in another batch.  The device computes the same function (csrc/sampling.cu).
"""
from __future__ import annotations

import struct

_MASK = (1 << 64) - 1


def mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_of(seed: int, seq_id: int, position: int) -> float:
    """A float32 value in [0, 1) with 24 random bits."""
    h = mix64(seed & _MASK)
    h = mix64(h ^ (seq_id & 0xFFFFFFFF))
    h = mix64(h ^ (position & 0xFFFFFFFF))
    return (h >> 40) / 16777216.0
