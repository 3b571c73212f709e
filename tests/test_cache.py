"""The cache's bookkeeping: slots and pages are never lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from titan_b200.cache import CacheError, CacheFull, CacheNeed, KVGroup, PagePool, SequenceCache, SlotAllocator, StateGroup


def make(max_tokens=1024, max_slots=6, max_context=512, window=100):
    needs = [CacheNeed("kv", 2, 16), CacheNeed("kv", 2, 16, window=window), CacheNeed("kv", 2, 16), None,
             CacheNeed("state", state_shape=(3, 4))]
    return SequenceCache(needs, max_tokens, max_slots, max_context, torch.float32, "cpu")


def test_lowest_free_first_and_reuse():
    a = SlotAllocator(3)
    assert [a.take(), a.take(), a.take()] == [0, 1, 2]
    with pytest.raises(CacheFull):
        a.take()
    a.give_back(1)
    a.give_back(0)
    assert a.take() == 0 and a.take() == 1
    a.check()


def test_double_free_and_unknown_ids():
    a = SlotAllocator(2)
    s = a.take()
    a.give_back(s)
    with pytest.raises(CacheError, match="twice"):
        a.give_back(s)
    with pytest.raises(CacheError, match="does not exist"):
        a.give_back(7)
    p = PagePool(4)
    with pytest.raises(CacheFull):
        p.take_many(5)
    assert p.free_count == 4          # nothing was taken


def test_groups_by_need():
    c = make()
    assert [type(g) for g in c.groups] == [KVGroup, KVGroup, StateGroup]
    assert c.groups[0].layers == [0, 2] and c.groups[1].layers == [1]
    assert c.layer_place == [(0, 0), (1, 0), (0, 1), None, (2, 0)]
    assert c.groups[0].storage.shape == (2, 2, 16, 2, 64, 16)          # layers, K/V, pages, heads, rows, dim
    assert c.groups[1].ring_rows == 128 and c.groups[1].table_width == 2
    assert c.groups[2].storage.shape == (1, 6, 3, 4)


def test_reserve_is_all_or_nothing():
    c = make(max_tokens=640)          # 10 pages
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve({a: 300})               # 5 pages in the full group, 2 in the ring
    with pytest.raises(CacheFull):
        c.reserve({a: 320, b: 330})   # 0 + 6 more pages: only 5 free
    assert c.groups[0].pool.held_count == 5 and b not in c.groups[0].pages_of
    c.reserve({b: 320})
    c.check()
    with pytest.raises(CacheFull, match="context"):
        c.reserve({a: 513})
    with pytest.raises(CacheError, match="not live"):
        c.reserve({5: 1})


def test_ring_group_stops_growing():
    c = make()
    s = c.alloc_slot()
    c.reserve({s: 500})
    assert len(c.groups[0].pages_of[s]) == 8 and len(c.groups[1].pages_of[s]) == 2
    assert c.groups[0].table[s, :8].tolist() == c.groups[0].pages_of[s]


def test_state_is_zeroed_on_alloc():
    c = make()
    s = c.alloc_slot()
    c.groups[2].storage[:, s] = 5.0
    c.free_slot(s)
    assert c.alloc_slot() == s and float(c.groups[2].storage[:, s].abs().sum()) == 0.0


def test_random_traffic_keeps_the_invariants():
    rng = random.Random(0)
    c = make(max_tokens=2048, max_slots=5, max_context=700)
    live = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.3 and len(live) < 5:
            live[c.alloc_slot()] = 0
        elif r < 0.5 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = live[s] + rng.randint(1, 90)
            try:
                c.reserve({s: n})
                c.commit(s, n)
                live[s] = n
            except CacheFull:
                pass
        c.check()
        assert c.tokens_held() == sum(-(-n // 64) * 64 for n in live.values())
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert all(g.pool.held_count == 0 for g in c.groups if isinstance(g, KVGroup))
    assert c.slots.free_count == 5
