"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from skyla_kernel_b200.cache import CacheError, CacheFull, FreeList, KVNeed, SequenceCache, StateNeed


def _cache(max_tokens=640, window=None, max_slots=None):
    needs = [KVNeed(2, 16), KVNeed(2, 16), KVNeed(1, 32, window)]
    states = [None, StateNeed((3,)), None]
    return SequenceCache(needs, states, max_tokens, max_slots, torch.float32, None)


def test_free_list_refuses_misuse():
    f = FreeList(3, "thing")
    a, b, c = f.take(), f.take(), f.take()
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(CacheFull):
        f.take()
    f.give_back(b)
    with pytest.raises(CacheError, match="freed twice"):
        f.give_back(b)
    with pytest.raises(CacheError, match="does not exist"):
        f.give_back(7)
    assert f.take() == 1  # the lowest free number comes back first
    f.check()


def test_groups_by_need():
    c = _cache()
    assert len(c.groups) == 2 and c.groups[0].n_layers == 2 and c.groups[1].n_layers == 1
    assert c.entry_group == [(0, 0), (0, 1), (1, 0)]
    assert c.n_pages == 10


def test_reserve_is_all_or_nothing_and_reports_full():
    c = _cache(max_tokens=256)  # 4 pages per group
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 100), (b, 64)])  # 2 + 1 pages
    c.advance([(a, 100), (b, 64)])
    with pytest.raises(CacheFull, match="cache full"):
        c.reserve([(a, 29), (b, 1)])  # a needs 1 more, b needs 1 more: only 1 free
    assert c.groups[0].pages.n_held == 3  # nothing changed
    c.reserve([(a, 28)])  # still inside a's second page
    c.check()
    with pytest.raises(CacheError, match="twice"):
        c.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError, match="not in use"):
        c.reserve([(5, 1)])


def test_free_twice_and_unknown_slot():
    c = _cache()
    s = c.alloc_slot()
    c.free_slot(s)
    with pytest.raises(CacheError):
        c.free_slot(s)
    with pytest.raises(CacheError):
        c.length(s)


def test_random_traffic_never_loses_anything():
    rng = random.Random(0)
    c = _cache(max_tokens=64 * 40, window=100, max_slots=12)
    live = {}
    for it in range(3000):
        op = rng.random()
        if op < 0.25 and c.slots.n_free:
            s = c.alloc_slot()
            assert s not in live
            live[s] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            batch = rng.sample(list(live), rng.randint(1, len(live)))
            growth = [(s, rng.choice([1, 1, 1, 7, 64, 130])) for s in batch]
            try:
                c.reserve(growth)
            except CacheFull:
                continue
            c.advance(growth)
            for s, n in growth:
                live[s] += n
        if it % 50 == 0:
            c.check()
            for s, n in live.items():
                assert c.length(s) == n
                full, win = c.groups[0], c.groups[1]
                assert len(full.slot_pages[s]) >= -(-n // 64)
                assert all(p >= 0 for p in full.slot_pages[s])
                # the windowed group holds only pages the next token can still see
                first = max(0, n - 100 + 1) // 64
                assert all((p >= 0) == (j >= first) for j, p in enumerate(win.slot_pages[s]))
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert c.slots.n_held == 0 and all(g.pages.n_held == 0 for g in c.groups)


def test_slots_are_reused_lowest_first():
    c = _cache()
    a, b, d = c.alloc_slot(), c.alloc_slot(), c.alloc_slot()
    c.free_slot(b)
    c.free_slot(a)
    assert c.alloc_slot() == a and c.alloc_slot() == b
    assert c.tokens_held() == 0


def test_state_area_is_zeroed_on_alloc():
    needs = [KVNeed(1, 16)]
    c = SequenceCache(needs, [StateNeed((4,))], 128, 2, torch.float32, "cpu")
    s = c.alloc_slot()
    c.state_of_entry(0)[s] += 5
    c.free_slot(s)
    assert c.alloc_slot() == s
    assert torch.equal(c.state_of_entry(0)[s], torch.zeros(4))


def test_needs_that_differ_only_in_precision_get_storage_of_their_own():
    import torch
    needs = [KVNeed(2, 16), KVNeed(2, 16, None, torch.float32), KVNeed(2, 16)]
    c = SequenceCache(needs, [None] * 3, 256, None, torch.bfloat16, "cpu")
    assert len(c.groups) == 2 and sorted(g.n_layers for g in c.groups) == [1, 2]
    assert {g.k.dtype for g in c.groups} == {torch.bfloat16, torch.float32}
    assert c.entry_group[0][0] == c.entry_group[2][0] != c.entry_group[1][0]
    assert c.bytes_per_token() == 2 * 2 * 16 * (2 * 2 + 1 * 4)
