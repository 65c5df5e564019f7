"""The cache's bookkeeping: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200.cache import Cache, CacheError, SlotAllocator
from longbow_quarrel_b200.parts.base import KVNeed, StateNeed


def test_slots_are_never_lost_or_held_twice():
    a = SlotAllocator(5)
    held = [a.alloc() for _ in range(5)]
    assert sorted(held) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheError, match="no free slot"):
        a.alloc()
    a.free(held[2])
    with pytest.raises(CacheError, match="freed twice"):
        a.free(held[2])
    with pytest.raises(CacheError, match="not live"):
        a.free(77)
    assert a.alloc() == held[2]          # a slot that was given back is used again
    rng = random.Random(0)
    live = set(held)
    for _ in range(2000):
        if live and (rng.random() < 0.5 or not a.n_free):
            s = rng.choice(sorted(live)); a.free(s); live.remove(s)
        else:
            s = a.alloc(); assert s not in live; live.add(s)
        assert a.n_live == len(live) and a.n_live + a.n_free == 5


def _cache(max_tokens=640, window=None, max_context=512, max_slots=None):
    needs = {0: KVNeed(2, 16), 1: KVNeed(2, 16), 2: KVNeed(2, 16, window) if window else KVNeed(2, 16),
             3: StateNeed((3, 4))}
    return Cache(needs, max_tokens, max_context, torch.float32, "cpu", max_slots=max_slots)


def test_groups_by_need():
    c = _cache(window=40)
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    full = next(g for g in c.kv_groups if g.window is None)
    win = next(g for g in c.kv_groups if g.window == 40)
    assert full.entries == [0, 1] and win.entries == [2]
    assert full.k_pages.shape == (2, 10, 2, 64, 16) and win.k_pages.shape == (1, 10, 2, 64, 16)
    assert c.view(0).k_pages.data_ptr() != c.view(1).k_pages.data_ptr()
    assert c.view(3).shape == (c.max_slots, 3, 4)
    assert c.view(9) is None


def test_pages_follow_each_sequences_own_length():
    c = _cache(max_tokens=640)           # 10 pages
    s0, s1 = c.alloc_slot(), c.alloc_slot()
    c.reserve(s0, 65); c.commit(s0, 65)          # 2 pages
    c.reserve(s1, 1); c.commit(s1, 1)            # 1 page
    g = c.kv_groups[0]
    assert len(g.pages_of(s0)) == 2 and len(g.pages_of(s1)) == 1 and c.pages_in_use() == 3
    assert not set(g.pages_of(s0)) & set(g.pages_of(s1))
    for _ in range(63):
        c.reserve(s1, 1); c.commit(s1, 1)
    assert c.length(s1) == 64 and len(g.pages_of(s1)) == 1
    c.reserve(s1, 1); c.commit(s1, 1)
    assert len(g.pages_of(s1)) == 2
    c.free_slot(s0)
    assert c.pages_in_use() == 2 and g.pages_of(s0) == []
    with pytest.raises(CacheError, match="not live"):
        c.reserve(s0, 1)
    with pytest.raises(CacheError):
        c.free_slot(s0)


def test_full_cache_and_context_limit_are_errors():
    c = _cache(max_tokens=256, max_context=512)      # 4 pages, context limited by them
    s0, s1 = c.alloc_slot(), c.alloc_slot()
    c.reserve(s0, 129); c.commit(s0, 129)            # 3 pages
    c.reserve(s1, 64); c.commit(s1, 64)              # 1 page
    with pytest.raises(CacheError, match="full"):
        c.reserve(s1, 1)
    c.free_slot(s0)
    c.reserve(s1, 1)
    c2 = _cache(max_tokens=6400, max_context=100)
    s = c2.alloc_slot()
    with pytest.raises(CacheError, match="context limit"):
        c2.reserve(s, 101)


def test_a_window_group_gives_pages_back_as_the_sequence_moves_on():
    c = _cache(max_tokens=64 * 40, window=40, max_context=2048)
    full = next(g for g in c.kv_groups if g.window is None)
    win = next(g for g in c.kv_groups if g.window == 40)
    s = c.alloc_slot()
    c.reserve(s, 300); c.commit(s, 300)
    assert len(full.pages_of(s)) == 5
    # a later token at position >= 300 sees keys from 261 on: pages 4.. (positions 256..)
    assert len(win.pages_of(s)) == 1 and win.table[s, 4] != -1
    for _ in range(400):
        c.reserve(s, 1); c.commit(s, 1)
        assert len(win.pages_of(s)) <= 2
        first = win.first_needed(c.length(s))
        assert win.table[s, first // 64] != -1
    assert len(full.pages_of(s)) == 11
    c.free_slot(s)
    assert c.pages_in_use() == 0


def test_random_traffic_never_loses_a_page():
    c = _cache(max_tokens=64 * 30, window=100, max_context=1000, max_slots=6)
    rng = random.Random(1)
    live = {}
    for _ in range(3000):
        r = rng.random()
        if r < 0.1 and len(live) < 6:
            live[c.alloc_slot()] = 0
        elif r < 0.15 and live:
            s = rng.choice(sorted(live)); c.free_slot(s); del live[s]
        elif live:
            s = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 5, 70])
            try:
                c.reserve(s, n)
            except CacheError:
                continue
            c.commit(s, n); live[s] += n
        for g in c.kv_groups:
            held = [p for s in range(c.max_slots) for p in g.pages_of(s)]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + g.n_free_pages == g.n_pages, "a page was lost"
            for s in range(c.max_slots):
                if s not in live:
                    assert g.pages_of(s) == []
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.free_slot(s)
    assert c.pages_in_use() == 0 and c.slots.n_free == 6


def test_state_is_zeroed_when_a_slot_is_handed_out():
    c = _cache()
    s = c.alloc_slot()
    c.view(3)[s] += 5.0
    c.free_slot(s)
    assert c.alloc_slot() == s
    assert float(c.view(3)[s].abs().sum()) == 0.0


def test_page_table_reaches_the_device_copy():
    c = _cache()
    s = c.alloc_slot()
    c.reserve(s, 130)
    g = c.kv_groups[0]
    assert int(g.table_dev[s, 0]) == -1
    c.upload()
    assert g.table_dev[s].tolist() == g.table[s].tolist() and g.table[s, 2] != -1
    c.free_slot(s); c.upload()
    assert set(g.table_dev[s].tolist()) == {-1}
