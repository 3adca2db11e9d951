"""Host-side bookkeeping of the cache: which pages and which slots are free.

The reference gives every sequence a whole cache of `max_seq_len` positions
(src/context.cpp:5-20; src/kv_cache.cpp:14-17).  Here memory is cut into pages of a fixed
number of tokens, a sequence holds only the pages its length needs, and both pages and
slots go back to their free lists when the sequence ends.  These two classes hold no
device memory; their invariants (nothing lost, held twice or freed twice) are what the
CPU tests check.
"""
from __future__ import annotations

import heapq
from typing import List, Set


class CacheFull(RuntimeError):
    """No free page or slot is left; the message says what was asked and what is free."""


class CacheMisuse(RuntimeError):
    """A page or slot was released that is not held, or used after release."""


class FreeList:
    """Ids 0..n-1, each either free or held.  Lowest free id first, so reuse is visible."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise ValueError(f"number of {what}s must not be negative")
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n))                  # a heap; the lowest id comes first
        self._held: Set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def held(self) -> Set[int]:
        return set(self._held)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what}: all {self.n} are held")
        i = heapq.heappop(self._free)
        self._held.add(i)
        return i

    def take_many(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}s asked for, {len(self._free)} of {self.n} free")
        return [self.take() for _ in range(count)]

    def give_back(self, i: int) -> None:
        if i not in self._held:
            raise CacheMisuse(f"{self.what} {i} is not held (released twice, or never taken)")
        self._held.remove(i)
        heapq.heappush(self._free, i)

    def check(self) -> None:
        """Every id is exactly once in free ∪ held."""
        if len(self._free) != len(set(self._free)):
            raise AssertionError(f"a {self.what} is on the free list twice")
        if set(self._free) & self._held:
            raise AssertionError(f"a {self.what} is both free and held")
        if len(self._free) + len(self._held) != self.n:
            raise AssertionError(f"{self.what}s lost: {len(self._free)} free + {len(self._held)} held != {self.n}")
