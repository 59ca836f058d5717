"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (CPU)."""
import random

import pytest

from llmi_b200.cache import CacheError, PagePool, SlotTable, pages_for


def test_slots_are_handed_out_once_and_reused():
    t = SlotTable(3)
    a, b, c = t.alloc(), t.alloc(), t.alloc()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheError, match="no free slot"):
        t.alloc()
    t.free(b)
    with pytest.raises(CacheError, match="freed twice"):
        t.free(b)
    with pytest.raises(CacheError, match="not live"):
        t.free(17)
    assert t.alloc() == b and t.live == {a, b, c}


def test_pages_grow_by_need_and_return_on_close():
    p = PagePool(6, 64)
    p.open(0)
    p.open(1)
    assert p.extend(0, 1) == 0 and len(p.table(0)) == 1
    assert p.extend(0, 63) == 1 and len(p.table(0)) == 1           # still one page
    assert p.extend(0, 1) == 64 and len(p.table(0)) == 2           # position 64 opens the second page
    assert p.extend(1, 200) == 0 and len(p.table(1)) == 4 and p.n_free == 0
    assert p.pages_needed(0, 64) == 1
    with pytest.raises(CacheError, match="cache is full"):
        p.extend(0, 64)
    assert p.length(0) == 65                                       # a refused growth changes nothing
    p.check()
    p.close(1)
    assert p.n_free == 4
    with pytest.raises(CacheError, match="not open"):
        p.close(1)
    with pytest.raises(CacheError, match="already open"):
        p.open(0)
    p.extend(0, 64)
    p.check()
    p.close(0)
    assert p.n_free == 6 and sorted(p._free) == list(range(6))


def test_window_gives_pages_back_early():
    p = PagePool(4, 64, window=100)
    p.open(0)
    p.extend(0, 64 * 3)                    # prompt of 192 tokens: three pages
    assert p.n_free == 1
    for _ in range(300):                   # long decoding never needs more than the window's pages
        p.extend(0, 1)
        p.check()
    table = p.table(0)
    assert table[0] == -1 and table[-1] >= 0
    first_needed = p.length(0) - 1 - 100 + 1
    assert all(pg >= 0 for pg in table[first_needed // 64:])
    assert sum(pg >= 0 for pg in table) <= pages_for(100 + 63) + 1


def test_random_walk_never_loses_a_page():
    rng = random.Random(4)
    pool, slots = PagePool(40, 64), SlotTable(8)
    live = {}
    for _ in range(3000):
        r = rng.random()
        if r < 0.25 and slots.n_free:
            s = slots.alloc()
            pool.open(s)
            live[s] = 0
        elif r < 0.4 and live:
            s = rng.choice(list(live))
            pool.close(s)
            slots.free(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 5, 64, 130])
            try:
                base = pool.extend(s, n)
                assert base == live[s]
                live[s] += n
            except CacheError:
                assert pool.pages_needed(s, n) > pool.n_free
        pool.check()
        held = sum(len(pool.table(s)) for s in live)
        assert held + pool.n_free == 40
        assert all(len(pool.table(s)) == pages_for(live[s]) for s in live)
    for s in list(live):
        pool.close(s)
        slots.free(s)
    assert pool.n_free == 40 and slots.n_free == 8
