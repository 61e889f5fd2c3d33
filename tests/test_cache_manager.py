"""Cache manager and prefix cache on the host (no GPU): no page lost, held twice or freed twice."""
import random

import numpy as np
import pytest

from llm_singularity_b200.cache import CacheManager, PageError, PagePool, NO_PAGE
from llm_singularity_b200.cache.prefix import RadixPrefixCache
from llm_singularity_b200.parts.base import PagedKVSpec, StateSpec


def test_pool_allocates_frees_exhausts():
    # the reference's pool test (tests/test_memory.cpp:4-25): allocate all, exhaust, free, reuse
    pool = PagePool(3)
    a, b, c = pool.allocate(), pool.allocate(), pool.allocate()
    assert sorted([a, b, c]) == [0, 1, 2] and pool.allocate() is None and pool.num_free == 0
    pool.release(b)
    assert pool.num_free == 1 and pool.allocate() == b


def test_pool_refuses_double_free_and_foreign_pages():
    pool = PagePool(2)
    p = pool.allocate()
    pool.release(p)
    with pytest.raises(PageError, match="twice"):
        pool.release(p)
    with pytest.raises(PageError, match="outside"):
        pool.release(5)
    with pytest.raises(PageError, match="free"):
        pool.retain(p)


def _manager(pages=8, page=4, slots=3, specs=None, max_pages=8):
    specs = specs or [PagedKVSpec(2, 16), PagedKVSpec(2, 16)]
    return CacheManager(specs, page, pages, slots, max_pages)


def test_reserve_is_all_or_nothing_and_pages_come_back():
    m = _manager(pages=4)
    assert m.open("a") == 0 and m.open("b") == 1
    assert m.reserve("a", 9) and m.pages_of("a") == [0, 1, 2]        # 3 pages of 4 tokens
    m.commit("a", 9)
    assert not m.reserve("b", 8)                                     # needs 2, 1 free
    assert m.pages_of("b") == [] and m.free_pages() == 1             # nothing was taken
    assert m.reserve("b", 4)
    m.commit("b", 4)
    m.check_invariants()
    m.close("a")
    assert m.free_pages() == 3 and m.reserve("b", 16)                # a's pages are used again
    assert set(m.pages_of("b")) == {0, 1, 2, 3}
    m.close("b")
    assert m.free_pages() == 4
    m.check_invariants()


def test_slots_run_out_and_return():
    m = _manager(slots=2)
    assert m.open("a") is not None and m.open("b") is not None and m.open("c") is None
    m.close("a")
    assert m.open("c") is not None
    with pytest.raises(KeyError):
        m.open("c")


def test_commit_needs_pages_and_tables_have_a_limit():
    m = _manager(pages=8, max_pages=2)
    m.open("a")
    with pytest.raises(PageError, match="not covered"):
        m.commit("a", 3)
    with pytest.raises(PageError, match="block table"):
        m.reserve("a", 9)


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    specs = [PagedKVSpec(2, 16), PagedKVSpec(2, 16, window=6), PagedKVSpec(1, 32, window=6),
             StateSpec((4,)), None]
    m = CacheManager(specs, 4, {None: 8, 6: 5}, 2, 8)
    assert len(m.groups) == 2 and m.groups[0].cache_ids == [0] and m.groups[1].cache_ids == [1, 2]
    m.open("a")
    full, win = m.groups[0], m.groups[1]
    for n in range(1, 29):
        assert m.reserve("a", n), n          # the window group never holds more than 3 pages
        m.commit("a", n)
        m.check_invariants()
    assert full.pool.num_used == 7
    # next query sits at 28 and sees keys 23..28: pages 0..4 (positions 0..19) are passed
    assert win.pool.num_used == 2 and list(win.table[0, :7]) == [NO_PAGE] * 5 + list(win.table[0, 5:7])
    assert all(p >= 0 for p in win.table[0, 5:7])
    m.close("a")
    assert full.pool.num_free == 8 and win.pool.num_free == 5
    m.check_invariants()


def test_table_updates_are_reported_once():
    m = _manager(pages=4, max_pages=8)
    m.open("a")
    m.reserve("a", 5)
    ups = m.take_updates(0)
    assert ups == [(0, 0), (1, 1)] and m.take_updates(0) == []
    m.close("a")
    assert m.take_updates(0) == [(0, NO_PAGE), (1, NO_PAGE)]


def test_table_updates_as_arrays_keep_the_last_value_of_a_cell():
    """A request that ends and another that takes its pages between two steps write the same cells
    twice: the arrays give every cell once, with its last value."""
    m = _manager(pages=4, max_pages=8)
    m.open("a")
    m.reserve("a", 5)
    m.close("a")
    m.open("b")
    m.reserve("b", 9)
    table = m.groups[0].table.copy()
    cells, values = m.take_update_arrays(0)
    assert len(set(cells.tolist())) == len(cells) == 3
    flat = np.full(table.size, NO_PAGE, dtype=np.int32)
    flat[cells] = values
    assert (flat.reshape(table.shape) == table).all()
    again = m.take_update_arrays(0)
    assert len(again[0]) == 0 and len(again[1]) == 0 and m.take_updates(0) == []


@pytest.mark.parametrize("seed", range(3))
def test_update_arrays_equal_the_pairs_with_later_writes_winning(seed):
    """Two managers driven alike under random opening, growing and closing of requests: the arrays
    of one are, as a mapping, the pairs of the other with later writes to a cell winning; also
    when hundreds of cells change between two calls."""
    rng = random.Random(seed)
    a, b = _manager(pages=64, max_pages=32, slots=6), _manager(pages=64, max_pages=32, slots=6)
    live = {}
    for step in range(300):
        for m in (a, b):
            m_rng = random.Random(seed * 1000 + step)
            op = m_rng.random()
            names = sorted(live)
            if op < 0.3 and len(live) < 6:
                name = f"r{step}"
                m.open(name)
                if m is b:
                    live[name] = 0
            elif op < 0.8 and names:
                name = names[m_rng.randrange(len(names))]
                grow = live[name] + m_rng.randrange(1, 60)
                if grow <= 32 * 4 and m.reserve(name, grow):
                    m.commit(name, grow)
                    if m is b:
                        live[name] = grow
            elif names:
                name = names[m_rng.randrange(len(names))]
                m.close(name)
                if m is b:
                    del live[name]
        if rng.random() < 0.15 or step == 299:
            pairs = dict(a.take_updates(0))
            cells, values = b.take_update_arrays(0)
            assert len(set(cells.tolist())) == len(cells)
            assert dict(zip(cells.tolist(), values.tolist())) == pairs
    a.check_invariants(); b.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    specs = [PagedKVSpec(1, 16), PagedKVSpec(1, 16, window=5)]
    m = CacheManager(specs, 4, {None: 12, 5: 6}, 4, 16)
    live = {}
    for step in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{step}"
            assert m.open(rid) is not None
            live[rid] = 0
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = live[rid] + rng.choice([1, 1, 1, 2, 3, 7])
            if n <= 64 and m.reserve(rid, n):
                m.commit(rid, n)
                live[rid] = n
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check_invariants()
        used = sum(-(-n // 4) for n in live.values())
        assert m.groups[0].pool.num_used >= used          # reserved-but-uncommitted pages allowed
    for rid in list(live):
        m.close(rid)
    m.check_invariants()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups)


# ------------------------------------------------------------------ prefix cache
def _finish(m, pc, rid, tokens):
    pc.insert(tokens, rid)
    m.close(rid)


def test_prefix_cache_shares_whole_pages_only_and_never_the_last_token():
    m = _manager(pages=8, page=4)
    pc = RadixPrefixCache(m)
    toks = list(range(100, 110))                      # 10 tokens: 2 full pages + 2
    m.open("a"); m.reserve("a", 10); m.commit("a", 10)
    pages_a = m.pages_of("a")
    _finish(m, pc, "a", toks)
    assert pc.num_nodes == 2 and m.free_pages() == 6  # the partial page went back
    m.check_invariants()
    # same prompt again (tests/test_scheduler.cpp:92-127 expects a hit): 2 pages adopted
    path = pc.match(toks)
    assert len(path) == 2
    m.open("b")
    assert pc.adopt("b", path) == 8 and m.pages_of("b") == pages_a[:2] and m.length("b") == 8
    # a prompt that is exactly the cached pages still recomputes its last page
    assert len(pc.match(toks[:8])) == 1
    # a longer query matches the stored prefix; a different start matches nothing
    assert len(pc.match(toks + [1, 2, 3])) == 2 and pc.match([9] + toks) == []
    m.check_invariants()
    assert pc.evictable_pages() == 0 and pc.evict(2) == 0      # in use: nothing to evict
    pc.release(path); m.close("b")
    assert pc.evictable_pages() == 2
    m.check_invariants()


def test_prefix_cache_evicts_leaves_first_least_recently_used():
    m = _manager(pages=8, page=4)
    pc = RadixPrefixCache(m)
    for rid, toks in (("a", [1] * 4 + [2] * 4 + [0]), ("b", [1] * 4 + [3] * 4 + [0]), ("c", [7] * 4 + [0])):
        m.open(rid); m.reserve(rid, len(toks)); m.commit(rid, len(toks))
        _finish(m, pc, rid, toks)
    assert pc.num_nodes == 4 and m.free_pages() == 4   # [1111] is stored once
    path = pc.match([1] * 4 + [2] * 4 + [5])           # touch a's branch: it becomes most recent
    m.open("d"); pc.adopt("d", path); pc.release(path); m.close("d")
    assert pc.evict(1) == 1                            # b's leaf [3333] is the oldest leaf
    assert len(pc.match([1] * 4 + [3] * 4 + [5])) == 1
    assert pc.evict(10) == 3 and pc.num_nodes == 0 and m.free_pages() == 8
    m.check_invariants()


def test_prefix_cache_needs_layers_that_keep_all_keys():
    m = CacheManager([PagedKVSpec(1, 16, window=4)], 4, 4, 2, 4)
    with pytest.raises(ValueError):
        RadixPrefixCache(m)
