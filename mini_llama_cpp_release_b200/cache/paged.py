"""The cache of a context: pages of keys and values per group of layers, a slot per
sequence, and fixed-size state per slot.

Layout of a group's pools (one for keys, one for values), in the engine's element type:
    [entries of the group][pages][kv_heads][page_size tokens][head_dim]
so the keys of one (page, kv head) are one dense block.  The reference's cache is
[layers][max_seq_len][kv_heads][head_dim] per sequence, zero-filled
(src/kv_cache.cpp:14-17, 41-45); nothing is zero-filled here because reads stop at each
sequence's own length.

A *group* collects the schedule entries whose mixers declared the same need (all keys,
or a window of them, with the same heads and head size); each group has its own pools,
its own free list and its own page lists, so a model whose layers need different things
stores each kind by itself.  A window group gives pages back as soon as every position in
them has left the window.

Beside the groups, every schedule entry whose mixer declared a `StateSpec` gets a tensor
[n_slots, *shape], zeroed when a slot is taken.  The architecture of this library
declares none; the area exists so that a mixer that needs it finds it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..kernels import KVView
from ..parts.base import CacheNeed, StateSpec
from .pool import CacheFull, CacheMisuse, FreeList

PAGE_SIZE = 64


@dataclass
class GroupLayout:
    need: CacheNeed
    entries: List[int]                 # schedule entries that own a cache in this group, in order

    def index_of(self, entry: int) -> int:
        return self.entries.index(entry)


def plan_groups(needs: Sequence[Optional[CacheNeed]], reads_cache_of: Sequence[Optional[int]]) -> Tuple[List[GroupLayout], List[Optional[Tuple[int, int]]]]:
    """From each schedule entry's need (None: keeps no keys) and sharing, the groups and, per
    entry, (group, index inside the group) of the cache it uses."""
    groups: List[GroupLayout] = []
    by_key: Dict[Tuple, int] = {}
    where: List[Optional[Tuple[int, int]]] = [None] * len(needs)
    for e, need in enumerate(needs):
        if need is None or reads_cache_of[e] is not None:
            continue
        g = by_key.get(need.group_key())
        if g is None:
            g = len(groups)
            by_key[need.group_key()] = g
            groups.append(GroupLayout(need, []))
        groups[g].entries.append(e)
        where[e] = (g, len(groups[g].entries) - 1)
    for e, src in enumerate(reads_cache_of):
        if src is not None:
            if where[src] is None:
                raise ValueError(f"schedule entry {e} reads the cache of entry {src}, which keeps none")
            if needs[e] is not None and needs[src] is not None and (
                    needs[e].kv_heads != needs[src].kv_heads or needs[e].head_dim != needs[src].head_dim):
                raise ValueError(f"schedule entry {e} cannot read the cache of entry {src}: kv heads or head size differ")
            if needs[e] is not None and needs[src] is not None and needs[src].kind == "window" and (
                    needs[e].kind != "window" or (needs[e].window or 0) > (needs[src].window or 0)):
                # the owner gives pages back once its own window has passed them; a reader that looks further back
                # would find them gone
                raise ValueError(f"schedule entry {e} cannot read the cache of entry {src}: it reads "
                                 f"{'all keys' if needs[e].kind != 'window' else f'a window of {needs[e].window}'}, "
                                 f"the owner keeps a window of {needs[src].window}")
            where[e] = where[src]
    return groups, where


def cache_bytes_per_token(needs: Sequence[Optional[CacheNeed]], reads_cache_of: Sequence[Optional[int]], itemsize: int) -> int:
    """Key and value bytes one token of one sequence occupies over all groups, for elements of `itemsize` bytes
    (a window group holds at most its window of them)."""
    groups, _ = plan_groups(needs, reads_cache_of)
    return sum(2 * len(g.entries) * g.need.kv_heads * g.need.head_dim * itemsize for g in groups)


class SlotBook:
    """Pure bookkeeping (no device memory): slots, each sequence's length and its pages in
    every group.  `PagedCache` adds the tensors."""

    def __init__(self, groups: Sequence[GroupLayout], max_tokens: int, max_seqs: int, page_size: int = PAGE_SIZE):
        if max_tokens <= 0:
            raise ValueError("the cache must hold at least one token")
        self.page_size = page_size
        self.n_pages = (max_tokens + page_size - 1) // page_size
        self.max_seqs = max(1, min(max_seqs, self.n_pages))
        self.groups = list(groups)
        self.slots = FreeList(self.max_seqs, "slot")
        self.pages = [FreeList(self.n_pages, f"page of group {g}") for g in range(len(self.groups))]
        self.length: Dict[int, int] = {}
        self.page_lists: Dict[int, List[List[int]]] = {}          # slot → per group → page per page index (-1: none)
        # slot → a number that changes whenever the slot's page lists change and is never used twice, so that whoever
        # keeps a copy of the lists (a captured decode step's page table on the device) can tell that it is stale,
        # also when the slot was given back and taken again in between
        self.page_version: Dict[int, int] = {}
        self._versions = 0

    # ---- slots
    def acquire(self) -> int:
        slot = self.slots.take()
        self.length[slot] = 0
        self.page_lists[slot] = [[] for _ in self.groups]
        self._touch(slot)
        return slot

    def _touch(self, slot: int) -> None:
        self._versions += 1
        self.page_version[slot] = self._versions

    def release(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheMisuse(f"slot {slot} is not held (released twice, or never taken)")
        for g, plist in enumerate(self.page_lists[slot]):
            for p in plist:
                if p >= 0:
                    self.pages[g].give_back(p)
        del self.page_lists[slot]
        del self.length[slot]
        del self.page_version[slot]
        self.slots.give_back(slot)

    def _require(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheMisuse(f"slot {slot} is not held")

    # ---- growth
    def reserve(self, slot: int, n_new: int) -> None:
        """Make room for n_new more tokens after the slot's current length (all groups)."""
        self._require(slot)
        new_len = self.length[slot] + n_new
        n_needed = (new_len + self.page_size - 1) // self.page_size
        lists = self.page_lists[slot]
        if all(len(pl) >= n_needed for pl in lists):         # the step of a decoded token, 63 times in 64
            return
        want = [max(0, n_needed - len(pl)) for pl in lists]
        for g, k in enumerate(want):
            if k > self.pages[g].n_free:
                raise CacheFull(
                    f"sequence in slot {slot} needs {k} more page(s) of {self.page_size} tokens in group {g}, "
                    f"{self.pages[g].n_free} of {self.n_pages} are free (the cache was sized for too few tokens)")
        for g, k in enumerate(want):
            self.page_lists[slot][g].extend(self.pages[g].take_many(k))
        if any(want):
            self._touch(slot)

    def reserve_all(self, wishes: Sequence[Tuple[int, int]]) -> None:
        """`reserve` for several (slot, n_new) at once: all of them, or none and `CacheFull`."""
        need = [0] * len(self.groups)
        for slot, n_new in wishes:
            self._require(slot)
            n_needed = (self.length[slot] + n_new + self.page_size - 1) // self.page_size
            for g, pl in enumerate(self.page_lists[slot]):
                need[g] += max(0, n_needed - len(pl))
        for g, k in enumerate(need):
            if k > self.pages[g].n_free:
                raise CacheFull(f"the batch needs {k} more page(s) of {self.page_size} tokens in group {g}, "
                                f"{self.pages[g].n_free} of {self.n_pages} are free (the cache was sized for too few tokens)")
        for slot, n_new in wishes:
            self.reserve(slot, n_new)

    def commit(self, slot: int, n_new: int) -> None:
        """The n_new tokens are in the cache now; drop pages a window has left behind."""
        self._require(slot)
        self.length[slot] += n_new
        L = self.length[slot]
        for g, layout in enumerate(self.groups):
            w = layout.need.window
            if layout.need.kind == "window" and w:
                first_needed = max(0, L - w + 1)                 # the next token reads keys from here on
                plist = self.page_lists[slot][g]
                for i in range(min(len(plist), first_needed // self.page_size)):
                    if plist[i] >= 0:
                        self.pages[g].give_back(plist[i])
                        plist[i] = -1
                        self._touch(slot)

    def tokens_held(self) -> int:
        """Tokens of live sequences, each rounded up to whole pages (the figure the cache is sized by)."""
        return sum(((n + self.page_size - 1) // self.page_size) * self.page_size for n in self.length.values())

    def check(self) -> None:
        self.slots.check()
        for g, fl in enumerate(self.pages):
            fl.check()
            held = [p for pl in self.page_lists.values() for p in pl[g] if p >= 0]
            if len(held) != len(set(held)):
                raise AssertionError(f"group {g}: a page is held by two sequences")
            if set(held) != fl.held():
                raise AssertionError(f"group {g}: pages held by sequences and by the free list disagree")
        if set(self.length) != self.slots.held():
            raise AssertionError("slots with a length and slots held disagree")


class PagedCache(SlotBook):
    """`SlotBook` plus the device tensors."""

    def __init__(self, needs: Sequence[Optional[CacheNeed]], reads_cache_of: Sequence[Optional[int]],
                 states: Sequence[Optional[StateSpec]], max_tokens: int, max_seqs: int, dtype: torch.dtype,
                 device: torch.device, page_size: int = PAGE_SIZE):
        groups, where = plan_groups(needs, reads_cache_of)
        super().__init__(groups, max_tokens, max_seqs, page_size)
        self.where = where
        self.dtype = dtype
        self.device = device
        self.k_pools: List[torch.Tensor] = []
        self.v_pools: List[torch.Tensor] = []
        for layout in groups:
            shape = (len(layout.entries), self.n_pages, layout.need.kv_heads, page_size, layout.need.head_dim)
            self.k_pools.append(torch.empty(shape, dtype=dtype, device=device))
            self.v_pools.append(torch.empty(shape, dtype=dtype, device=device))
        self.state: List[Optional[torch.Tensor]] = [
            torch.zeros((self.max_seqs, *s.shape), dtype=s.dtype, device=device) if s is not None else None
            for s in states]
        self.has_state = any(s is not None for s in self.state)

    def acquire(self) -> int:
        slot = super().acquire()
        for s in self.state:
            if s is not None:
                s[slot].zero_()
        return slot

    def snapshot_state(self, slots_long: torch.Tensor) -> List[Optional[torch.Tensor]]:
        """Copies of the given slots' rows of every state area; `restore_state` puts them back.  A step that is run
        once to warm up before it is captured into a graph, and then replayed, would otherwise advance its
        sequences' state twice (keys and values are written to the same places both times; state is not)."""
        if not self.has_state:
            return []
        return [s.index_select(0, slots_long) if s is not None else None for s in self.state]

    def restore_state(self, saved: Sequence[Optional[torch.Tensor]], slots_long: torch.Tensor) -> None:
        for s, rows in zip(self.state, saved):
            if s is not None:
                s.index_copy_(0, slots_long, rows)

    def bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in self.k_pools + self.v_pools)
        return n + sum(s.numel() * s.element_size() for s in self.state if s is not None)

    def bytes_per_token(self) -> int:
        """Key and value bytes one token of one sequence occupies over all groups."""
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.need.kv_heads * g.need.head_dim * item for g in self.groups)

    def view(self, entry: int, page_tables: Sequence[torch.Tensor]) -> Optional[KVView]:
        """The cache of schedule entry `entry` for the sequences whose page lists (one tensor
        per group, [n_seqs, pages]) are given."""
        w = self.where[entry]
        if w is None:
            return None
        g, idx = w
        need = self.groups[g].need
        per_entry = self.n_pages * need.kv_heads * self.page_size * need.head_dim
        return KVView(self.k_pools[g], self.v_pools[g], idx * per_entry, page_tables[g], self.page_size,
                      need.kv_heads, need.head_dim)
