"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (CPU)."""
import random

import pytest

from mini_llama_cpp_release_b200.cache import CacheFull, CacheMisuse, FreeList, GroupLayout, SlotBook, plan_groups
from mini_llama_cpp_release_b200.parts.base import CacheNeed

ALL = CacheNeed("all", 2, 16)
WIN = CacheNeed("window", 2, 16, window=100)


def test_free_list_gives_lowest_id_first_and_refuses_misuse():
    fl = FreeList(4, "slot")
    assert [fl.take() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        fl.take()
    fl.give_back(2)
    fl.give_back(0)
    with pytest.raises(CacheMisuse):
        fl.give_back(0)
    with pytest.raises(CacheMisuse):
        fl.give_back(7)
    assert fl.take() == 0 and fl.take() == 2
    fl.check()


def test_groups_collect_entries_with_the_same_need():
    needs = [ALL, WIN, ALL, None, WIN, ALL]
    groups, where = plan_groups(needs, [None, None, None, None, None, 0])
    assert [g.need for g in groups] == [ALL, WIN] and groups[0].entries == [0, 2] and groups[1].entries == [1, 4]
    assert where == [(0, 0), (1, 0), (0, 1), None, (1, 1), (0, 0)]
    with pytest.raises(ValueError, match="keeps none"):
        plan_groups([None, ALL], [None, 0])
    with pytest.raises(ValueError, match="differ"):
        plan_groups([ALL, CacheNeed("all", 4, 16)], [None, 0])


def book(max_tokens=64 * 10, max_seqs=4, groups=None):
    return SlotBook(groups or [GroupLayout(ALL, [0, 1])], max_tokens, max_seqs)


def test_pages_follow_length_and_come_back_on_release():
    b = book()
    s = b.acquire()
    b.reserve(s, 65); b.commit(s, 65)
    assert b.page_lists[s][0] == [0, 1] and b.length[s] == 65 and b.tokens_held() == 128
    b.reserve(s, 63); b.commit(s, 63)
    assert b.page_lists[s][0] == [0, 1]
    b.reserve(s, 1); b.commit(s, 1)
    assert b.page_lists[s][0] == [0, 1, 2]
    t = b.acquire()
    b.reserve(t, 1); b.commit(t, 1)
    assert b.page_lists[t][0] == [3]
    b.release(s)
    assert b.pages[0].n_free == 9
    with pytest.raises(CacheMisuse):
        b.release(s)
    with pytest.raises(CacheMisuse):
        b.reserve(s, 1)
    u = b.acquire()
    assert u == s                                   # the slot is used again
    b.reserve(u, 1)
    assert b.page_lists[u][0] == [0]                # and so is its page
    b.check()


def test_full_cache_says_what_is_missing_and_takes_nothing():
    b = book(max_tokens=64 * 3)
    s = b.acquire()
    b.reserve(s, 128); b.commit(s, 128)
    with pytest.raises(CacheFull, match="needs 3 more"):
        b.reserve(s, 130)
    assert b.pages[0].n_free == 1
    for _ in range(2):
        b.acquire()
    with pytest.raises(CacheFull, match="slot"):
        b.acquire()                                 # max_seqs is capped by the pages: 3
    b.check()


def test_window_group_gives_pages_back_as_they_leave_the_window():
    b = book(max_tokens=64 * 8, groups=[GroupLayout(ALL, [0]), GroupLayout(WIN, [1])])
    s = b.acquire()
    b.reserve(s, 300); b.commit(s, 300)
    # next token (position 300) reads keys from 201 on: pages 0..2 (positions < 192) are gone
    assert b.page_lists[s][1] == [-1, -1, -1, 3, 4] and b.page_lists[s][0] == [0, 1, 2, 3, 4]
    assert b.pages[1].n_free == 8 - 2 and b.pages[0].n_free == 3
    b.check()
    b.release(s)
    assert b.pages[1].n_free == 8 and b.pages[0].n_free == 8
    b.check()


def test_random_traffic_keeps_the_invariants():
    rng = random.Random(3)
    b = book(max_tokens=64 * 40, max_seqs=9, groups=[GroupLayout(ALL, [0]), GroupLayout(CacheNeed("window", 1, 8, 70), [1])])
    live = []
    for _ in range(2000):
        op = rng.random()
        try:
            if op < 0.25 and len(live) < 9:
                live.append(b.acquire())
            elif op < 0.45 and live:
                b.release(live.pop(rng.randrange(len(live))))
            elif live:
                s = rng.choice(live)
                n = rng.choice([1, 1, 1, 5, 64, 130])
                b.reserve(s, n)
                b.commit(s, n)
        except CacheFull:
            pass
        b.check()
    for s in live:
        b.release(s)
    b.check()
    assert b.slots.n_free == 9 and all(p.n_free == 40 for p in b.pages)


def test_a_reader_must_not_look_further_back_than_the_owner_keeps():
    """A run of the schedule that reads another run's cache finds only what the owner keeps: a window group gives
    pages back as positions leave its window."""
    narrow = CacheNeed("window", 2, 16, window=50)
    plan_groups([WIN, narrow], [None, 0])                        # a narrower window inside the owner's: fine
    plan_groups([ALL, WIN], [None, 0])                           # the owner keeps everything: fine
    with pytest.raises(ValueError, match="all keys"):
        plan_groups([WIN, ALL], [None, 0])
    with pytest.raises(ValueError, match="window of 100"):
        plan_groups([narrow, WIN], [None, 0])


def test_page_version_changes_with_every_change_of_a_slots_pages_and_is_never_used_twice():
    b = book(groups=[GroupLayout(ALL, [0]), GroupLayout(CacheNeed("window", 2, 16, window=70), [1])])
    s = b.acquire()
    seen = {b.page_version[s]}

    def changed():
        v = b.page_version[s]
        fresh = v not in seen
        seen.add(v)
        return fresh
    b.reserve(s, 60)
    assert changed()
    b.commit(s, 60)
    assert not changed()
    b.reserve(s, 1)
    b.commit(s, 1)
    assert not changed()                                         # 61 tokens: the same page
    b.reserve(s, 10)
    assert changed()                                             # a second page
    b.commit(s, 10)
    b.reserve(s, 70)
    b.commit(s, 70)
    assert changed()                                             # a third page came and the window let the first go
    # given back and taken again by another sequence of the same length: the same slot, the same number of pages,
    # another version
    other = b.acquire()
    b.reserve(other, 141)
    b.release(s)
    again = b.acquire()
    assert again == s
    b.reserve(again, 141)
    assert changed()
    b.check()
