"""The native memory layer (csrc/host_memory.cpp) against the plain one in Python
(tests/plain_memory.py): the same random operations on both, and everything they hand out must be
the same: slots, page ids, changed table cells, matched prefixes, evictions, refusals."""
import random

import pytest

import plain_memory
from llm_singularity_b200.cache import CacheManager, PageError
from llm_singularity_b200.cache.prefix import RadixPrefixCache
from llm_singularity_b200.parts.base import PagedKVSpec, StateSpec


def _pair(specs, page, pages, slots, max_pages, sharing):
    a = CacheManager(specs, page, pages, slots, max_pages)
    b = plain_memory.PlainCacheManager(specs, page, pages, slots, max_pages)
    return (a, RadixPrefixCache(a) if sharing else None), (b, plain_memory.PlainPrefixCache(b) if sharing else None)


def _same_state(a, b):
    assert a.live_requests() == b.live_requests() and a.free_pages() == b.free_pages()
    for gi in range(len(a.groups)):
        assert (a.groups[gi].table == b.groups[gi].table).all()
        assert a.take_updates(gi) == b.take_updates(gi)
        for r in a.live_requests():
            assert a.pages_of(r, gi) == b.pages_of(r, gi) and a.length(r) == b.length(r)
        for p in range(a.groups[gi].pool.num_pages):
            assert a.groups[gi].pool.refcount(p) == b.groups[gi].pool.refcount(p)


@pytest.mark.parametrize("seed", range(6))
def test_windows_and_groups_under_random_orders(seed):
    rng = random.Random(seed)
    specs = [PagedKVSpec(2, 16), PagedKVSpec(2, 16, window=rng.choice([3, 6, 9])), StateSpec((4,)), None,
             PagedKVSpec(1, 32)]
    (a, _), (b, _) = _pair(specs, rng.choice([2, 4]), {None: 12, specs[1].window: 7}, 3, 10, False)
    names = iter(range(10 ** 6))
    for _ in range(400):
        live = a.live_requests()
        op = rng.random()
        if op < 0.2 or not live:
            n = next(names)
            assert a.open(n) == b.open(n)
        elif op < 0.75:
            r = rng.choice(live)
            new = a.length(r) + rng.choice([1, 1, 2, 5, 9])
            try:
                got = a.reserve(r, new)
            except PageError:
                with pytest.raises(plain_memory.PageError):
                    b.reserve(r, new)
                continue
            assert got == b.reserve(r, new)
            if got:
                a.commit(r, new)
                b.commit(r, new)
        else:
            r = rng.choice(live)
            a.close(r)
            b.close(r)
        _same_state(a, b)
        a.check_invariants()
        b.check_invariants()
    for r in a.live_requests():
        a.close(r)
    assert all(g.pool.num_free == g.pool.num_pages for g in a.groups)


@pytest.mark.parametrize("seed", range(6))
def test_prefix_tree_under_random_orders(seed):
    rng = random.Random(100 + seed)
    page = rng.choice([2, 4])
    (a, ta), (b, tb) = _pair([PagedKVSpec(2, 16), PagedKVSpec(1, 32)], page, 24, 4, 24, True)
    tokens, paths = {}, {}
    stems = [[rng.randrange(3) for _ in range(40)] for _ in range(3)]     # few token values: shared prefixes
    names = iter(range(10 ** 6))
    for _ in range(500):
        live = a.live_requests()
        op = rng.random()
        if (op < 0.25 or not live) and len(live) < 4:
            n = next(names)
            toks = rng.choice(stems)[:rng.randrange(1, 40)] + [rng.randrange(3) for _ in range(rng.randrange(0, 6))]
            pa, pb = ta.match(toks), tb.match(toks)
            assert len(pa) == len(pb) and [x.pages for x in pa] == [x.pages for x in pb]
            assert ta.idle_on(pa) == sum(1 for x in pb if x.users == 0)
            assert a.open(n) == b.open(n)
            assert ta.adopt(n, pa) == tb.adopt(n, pb)
            tokens[n], paths[n] = toks, (pa, pb)
        elif op < 0.6:
            r = rng.choice(live)                       # run some more of its tokens
            new = min(len(tokens[r]), a.length(r) + rng.choice([1, 3, 7]))
            got = a.reserve(r, new)
            assert got == b.reserve(r, new)
            if not got:
                need = a.pages_needed(r, new) - a.free_pages()
                assert need == b.pages_needed(r, new) - b.free_pages()
                assert ta.evict(need) == tb.evict(need)
                got = a.reserve(r, new)
                assert got == b.reserve(r, new)
            if got:
                a.commit(r, new)
                b.commit(r, new)
        elif op < 0.75:
            r = rng.choice(live)                       # share what it has so far with later prompts
            pa, pb = paths[r]
            more_a = ta.share(tokens[r][:a.length(r)], r, pa)
            more_b = tb.share(tokens[r][:b.length(r)], r, pb)
            assert [x.pages for x in more_a] == [x.pages for x in more_b]
            paths[r] = (pa + more_a, pb + more_b)
        else:
            r = rng.choice(live)                       # it ends and leaves its full pages behind
            assert ta.insert(tokens[r][:a.length(r)], r) == tb.insert(tokens[r][:b.length(r)], r)
            pa, pb = paths.pop(r)
            ta.release(pa)
            tb.release(pb)
            a.close(r)
            b.close(r)
        assert ta.num_nodes == tb.num_nodes and ta.evictable_pages() == tb.evictable_pages()
        assert ta.hits == tb.hits
        _same_state(a, b)
        a.check_invariants()
        b.check_invariants()
        tb.check_invariants()
    for r in a.live_requests():
        ta.release(paths[r][0])
        a.close(r)
    ta.evict(10 ** 6)
    assert ta.num_nodes == 0 and a.free_pages() == 24
    a.check_invariants()


def test_the_memory_layer_refuses_what_would_corrupt_it():
    a = CacheManager([PagedKVSpec(2, 16)], 4, 8, 2, 4)
    tree = RadixPrefixCache(a)
    a.open("x")
    assert a.reserve("x", 8)
    a.commit("x", 8)
    assert tree.insert([1, 2, 3, 4, 5, 6, 7, 8], "x") == 2
    path = tree.match([1, 2, 3, 4, 5, 6, 7, 8, 9])
    assert len(path) == 2
    with pytest.raises(PageError, match="no user"):
        tree.release(path)                                   # nobody adopted it
    a.open("y")
    assert tree.adopt("y", path) == 8
    with pytest.raises(PageError, match="fresh request"):
        tree.adopt("y", path)                                # y already has pages
    a.check_invariants()
    with pytest.raises(ValueError, match="all its keys"):
        RadixPrefixCache(CacheManager([PagedKVSpec(2, 16, window=8)], 4, 8, 2, 4))
    with pytest.raises(ValueError):
        CacheManager([PagedKVSpec(2, 16)], 4, 0, 2, 4)
