"""A plain memory layer in Python: page pool, block tables per group, request slots and the prefix
tree, each with lists and dicts.  The engine's memory layer is native code
(``llm_singularity_b200/csrc/host_memory.cpp``); the tests drive both with the same random
operations and compare what they hand out.  It shares no code with the product and keeps no
device tensors."""
from __future__ import annotations

import itertools
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

NO_PAGE = -1


class PageError(RuntimeError):
    pass


class PlainPagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        # stack: the page freed last is handed out first; fresh pool pops 0, 1, 2, ...
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._refs: List[int] = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> Optional[int]:
        """A free page with one reference, or ``None`` if the pool is empty."""
        if not self._free:
            return None
        p = self._free.pop()
        assert self._refs[p] == 0
        self._refs[p] = 1
        return p

    def retain(self, page: int) -> None:
        self._check(page)
        if self._refs[page] == 0:
            raise PageError(f"page {page} is free and cannot be retained")
        self._refs[page] += 1

    def release(self, page: int) -> bool:
        """Drop one reference; returns True if the page went back to the free list."""
        self._check(page)
        if self._refs[page] == 0:
            raise PageError(f"page {page} freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)
            return True
        return False

    def refcount(self, page: int) -> int:
        self._check(page)
        return self._refs[page]

    def _check(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise PageError(f"page id {page} outside pool of {self.num_pages}")

    def check_invariants(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (self._refs[p] == 0) != (p in free):
                raise PageError(f"page {p}: refcount {self._refs[p]} disagrees with free list")


class _Group:
    def __init__(self, window: Optional[int], num_pages: int, slots: int, max_pages: int):
        self.window = window
        self.pool = PlainPagePool(num_pages)
        self.cache_ids: List[int] = []
        self.table = np.full((slots, max_pages), NO_PAGE, dtype=np.int32)   # host mirror
        self.updates: List[Tuple[int, int]] = []       # (flat index, value) not yet on device
        # per request: pages [0, first_live) have been released behind the window
        self.first_live: Dict[Hashable, int] = {}


class _Request:
    __slots__ = ("slot", "length", "num_pages")

    def __init__(self, slot: int):
        self.slot = slot
        self.length = 0
        self.num_pages = 0     # logical pages covered so far (same count in every group)


class PlainCacheManager:
    def __init__(self, cache_specs: Sequence[object], page_size: int, num_pages,
                 max_requests: int, max_pages_per_request: int):
        """``cache_specs[i]`` is what cache id ``i`` holds (PagedKVSpec, StateSpec or None);
        ``num_pages`` is an int (every group gets that many) or ``{window: pages}``."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_pages = max_pages_per_request
        self.groups: List[_Group] = []
        self._group_of: Dict[int, int] = {}
        self._specs = list(cache_specs)
        self._requests: Dict[Hashable, _Request] = {}
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))

        by_window: Dict[Optional[int], int] = {}
        for cid, cs in enumerate(self._specs):
            if hasattr(cs, "window"):
                if cs.window not in by_window:
                    n = num_pages[cs.window] if isinstance(num_pages, dict) else num_pages
                    by_window[cs.window] = len(self.groups)
                    self.groups.append(_Group(cs.window, n, max_requests, max_pages_per_request))
                g = by_window[cs.window]
                self.groups[g].cache_ids.append(cid)
                self._group_of[cid] = g
            elif not (cs is None or hasattr(cs, "shape")):
                raise TypeError(f"cache {cid}: unknown cache spec {cs!r}")

    # ---------------------------------------------------------------- requests
    def has(self, request: Hashable) -> bool:
        return request in self._requests

    def open(self, request: Hashable) -> Optional[int]:
        """Give ``request`` a slot (block-table row and state row); None if all are taken."""
        if request in self._requests:
            raise KeyError(f"request {request!r} is already open")
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._requests[request] = _Request(slot)
        for g in self.groups:
            g.first_live[request] = 0
        return slot

    def slot(self, request: Hashable) -> int:
        return self._requests[request].slot

    def length(self, request: Hashable) -> int:
        return self._requests[request].length

    def pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def pages_needed(self, request: Hashable, new_length: int) -> int:
        """Pages each group must still hand out to cover ``new_length`` tokens."""
        r = self._requests[request]
        return max(0, self.pages_for(new_length) - r.num_pages)

    def free_pages(self) -> int:
        """Pages free in the tightest group."""
        return min((g.pool.num_free for g in self.groups), default=1 << 30)

    def reserve(self, request: Hashable, new_length: int) -> bool:
        """Cover positions ``[0, new_length)`` with pages in every group, or change nothing."""
        r = self._requests[request]
        want = self.pages_for(new_length)
        if want > self.max_pages:
            raise PageError(f"request {request!r}: {new_length} tokens need {want} pages, "
                            f"a block table holds {self.max_pages}")
        need = want - r.num_pages
        if need <= 0:
            return True
        if any(g.pool.num_free < need for g in self.groups):
            return False
        for g in self.groups:
            for i in range(r.num_pages, want):
                page = g.pool.allocate()
                self._set(g, r.slot, i, page)
        r.num_pages = want
        return True

    def commit(self, request: Hashable, new_length: int) -> None:
        """The request now holds ``new_length`` tokens; give back pages a window has passed."""
        r = self._requests[request]
        if self.pages_for(new_length) > r.num_pages:
            raise PageError(f"request {request!r}: length {new_length} is not covered by its pages")
        r.length = new_length
        for g in self.groups:
            if g.window is None:
                continue
            # the next query sits at position >= new_length and sees keys > pos - window
            first_needed = max(0, new_length - g.window + 1)
            dead = min(first_needed // self.page_size, r.num_pages)
            for i in range(g.first_live[request], dead):
                g.pool.release(int(g.table[r.slot, i]))
                self._set(g, r.slot, i, NO_PAGE)
            g.first_live[request] = max(g.first_live[request], dead)

    def close(self, request: Hashable) -> None:
        """The request is over: every page it holds and its slot go back."""
        r = self._requests.pop(request)
        for g in self.groups:
            for i in range(g.first_live.pop(request), r.num_pages):
                g.pool.release(int(g.table[r.slot, i]))
                self._set(g, r.slot, i, NO_PAGE)
        self._free_slots.append(r.slot)

    def adopt(self, request: Hashable, pages_per_group: Sequence[Sequence[int]], length: int) -> None:
        """Start a fresh request on pages that already hold its first ``length`` tokens
        (shared through the prefix cache); takes one reference on each."""
        r = self._requests[request]
        if r.num_pages or length % self.page_size:
            raise PageError("adopt needs a fresh request and a whole number of pages")
        n = length // self.page_size
        for g, pages in zip(self.groups, pages_per_group):
            if len(pages) != n:
                raise PageError("adopt: page list does not match the length")
            for i, p in enumerate(pages):
                g.pool.retain(p)
                self._set(g, r.slot, i, p)
        r.num_pages = n
        r.length = length

    def pages_of(self, request: Hashable, group: int = 0) -> List[int]:
        r = self._requests[request]
        return [int(p) for p in self.groups[group].table[r.slot, :r.num_pages]]

    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    # ------------------------------------------------------------------ tables
    def _set(self, g: _Group, slot: int, index: int, page: int) -> None:
        g.table[slot, index] = page
        g.updates.append((slot * self.max_pages + index, page))

    def take_updates(self, group: int) -> List[Tuple[int, int]]:
        """Block-table cells changed since the last call, as (flat index, value)."""
        g = self.groups[group]
        ups, g.updates = g.updates, []
        return ups

    # -------------------------------------------------------------- invariants
    def check_invariants(self) -> None:
        """No page lost, none held twice by different owners without a reference, none freed twice."""
        for g in self.groups:
            g.pool.check_invariants()
            held: Dict[int, int] = {}
            for req, r in self._requests.items():
                for i in range(r.num_pages):
                    p = int(g.table[r.slot, i])
                    if i < g.first_live[req]:
                        if p != NO_PAGE:
                            raise PageError(f"released cell still names page {p}")
                        continue
                    if p == NO_PAGE:
                        raise PageError(f"request {req!r} lacks page {i}")
                    held[p] = held.get(p, 0) + 1
                if (g.table[r.slot, r.num_pages:] != NO_PAGE).any():
                    raise PageError(f"request {req!r}: cells past its pages are set")
            for p, n in held.items():
                if g.pool.refcount(p) < n:
                    raise PageError(f"page {p} held {n} times with refcount {g.pool.refcount(p)}")
            self._extra_refs_ok(g, held)
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PageError("a slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise PageError("a slot was lost")

    def _extra_refs_ok(self, g: _Group, held: Dict[int, int]) -> None:
        # references beyond those of live requests belong to the prefix cache, which
        # registers them here so that nothing is lost
        extra = getattr(self, "external_refs", None)
        for p in range(g.pool.num_pages):
            n = held.get(p, 0) + (extra(self.groups.index(g), p) if extra else 0)
            if g.pool.refcount(p) != n:
                raise PageError(f"page {p}: refcount {g.pool.refcount(p)} but {n} owners known")


class _Node:
    __slots__ = ("key", "pages", "children", "parent", "users", "last_used")

    def __init__(self, key, pages, parent):
        self.key: Tuple[int, ...] = key
        self.pages: Tuple[int, ...] = pages          # one page id per cache group
        self.children: Dict[Tuple[int, ...], "_Node"] = {}
        self.parent: Optional["_Node"] = parent
        self.users = 0                               # live requests whose prefix runs through here
        self.last_used = 0


class PlainPrefixCache:
    def __init__(self, cache: PlainCacheManager):
        if any(g.window is not None for g in cache.groups):
            raise ValueError("prefix sharing needs every layer to keep all its keys")
        self.cache = cache
        self.page_size = cache.page_size
        self.root = _Node((), (), None)
        self._clock = itertools.count(1)
        self.num_nodes = 0
        self.hits = 0                                # pages adopted instead of recomputed
        self._idle = 0                               # nodes no live request uses (kept up to date)
        cache.external_refs = self._owns

    # ---------------------------------------------------------------- lookup
    def match(self, tokens: Sequence[int]) -> List[_Node]:
        """Nodes of the longest cached prefix of ``tokens`` (whole pages, never the last token)."""
        ps = self.page_size
        limit = (len(tokens) - 1) // ps
        node, path = self.root, []
        for i in range(limit):
            child = node.children.get(tuple(tokens[i * ps:(i + 1) * ps]))
            if child is None:
                break
            path.append(child)
            node = child
        return path

    def adopt(self, request, path: List[_Node]) -> int:
        """Start ``request`` (open, no pages yet) on the pages of ``path``; returns tokens covered."""
        if not path:
            return 0
        now = next(self._clock)
        for n in path:
            if n.users == 0:
                self._idle -= 1
            n.users += 1
            n.last_used = now
        per_group = [[n.pages[g] for n in path] for g in range(len(self.cache.groups))]
        self.cache.adopt(request, per_group, len(path) * self.page_size)
        self.hits += len(path)
        return len(path) * self.page_size

    def release(self, path: List[_Node]) -> None:
        """The request that adopted ``path`` is gone (its page references are dropped by close)."""
        now = next(self._clock)
        for n in path:
            n.users -= 1
            if n.users == 0:
                self._idle += 1
            n.last_used = now

    # ---------------------------------------------------------------- insert
    def insert(self, tokens: Sequence[int], request) -> int:
        """Keep the full pages of ``request`` (which holds ``tokens``) for later prompts.
        Call before the request is closed.  Returns the number of pages newly kept."""
        ps = self.page_size
        n_full = min(len(tokens), self.cache.length(request)) // ps
        pages = [self.cache.pages_of(request, g) for g in range(len(self.cache.groups))]
        node, kept, now = self.root, 0, next(self._clock)
        for i in range(n_full):
            key = tuple(tokens[i * ps:(i + 1) * ps])
            child = node.children.get(key)
            if child is None:
                mine = tuple(pages[g][i] for g in range(len(pages)))
                for g, p in enumerate(mine):
                    self.cache.groups[g].pool.retain(p)
                child = _Node(key, mine, node)
                node.children[key] = child
                self.num_nodes += 1
                self._idle += 1
                kept += 1
            child.last_used = now
            node = child
        return kept

    def share(self, tokens: Sequence[int], request, held: Sequence[_Node]) -> List[_Node]:
        """Like :meth:`insert`, for a request that goes on running: the pages its ``tokens`` fill
        become visible to later prompts now (a prompt that arrives while this one still decodes
        need not recompute what they have in common).  ``held``: the nodes the request already counts
        as a user of (its adopted prefix).  Returns the further nodes whose pages are the
        request's own; it is a user of those too until :meth:`release`, so that they are not
        offered for eviction while evicting them would free nothing."""
        ps = self.page_size
        pages = [self.cache.pages_of(request, g) for g in range(len(self.cache.groups))]
        # (the step that fills these pages may only be planned yet: whoever reads them is queued
        # behind it, so the pages count as full as soon as they are the request's)
        n_full = min([len(tokens) // ps] + [len(p) for p in pages])
        mine_of = lambda i: tuple(pages[g][i] for g in range(len(pages)))
        have = set(map(id, held))
        node, now, added = self.root, next(self._clock), []
        for i in range(n_full):
            key = tuple(tokens[i * ps:(i + 1) * ps])
            mine = mine_of(i)
            child = node.children.get(key)
            if child is None:
                for g, p in enumerate(mine):
                    self.cache.groups[g].pool.retain(p)
                child = _Node(key, mine, node)
                node.children[key] = child
                self.num_nodes += 1
                self._idle += 1
            child.last_used = now
            if child.pages == mine and id(child) not in have:
                if child.users == 0:
                    self._idle -= 1
                child.users += 1
                added.append(child)
            node = child
        return added

    # -------------------------------------------------------------- eviction
    def evictable_pages(self) -> int:
        return self._idle

    def evict(self, pages_wanted: int) -> int:
        """Give back up to ``pages_wanted`` pages per group; returns how many were freed."""
        freed = 0
        while freed < pages_wanted:
            leaves = [n for n in self._nodes() if not n.children and n.users == 0]
            if not leaves:
                break
            leaves.sort(key=lambda n: n.last_used)
            for n in leaves:
                if freed >= pages_wanted:
                    break
                for g, p in enumerate(n.pages):
                    self.cache.groups[g].pool.release(p)
                del n.parent.children[n.key]
                self.num_nodes -= 1
                self._idle -= 1
                freed += 1
        return freed

    def check_invariants(self) -> None:
        """The counters agree with the tree (tests call this)."""
        nodes = list(self._nodes())
        if len(nodes) != self.num_nodes or sum(1 for n in nodes if n.users == 0) != self._idle:
            raise AssertionError(f"prefix tree: {len(nodes)} nodes / {self.num_nodes} counted, "
                                 f"{sum(1 for n in nodes if n.users == 0)} idle / {self._idle} counted")
        if any(n.users < 0 for n in nodes):
            raise AssertionError("prefix tree: a node has fewer than zero users")

    def _nodes(self):
        stack = list(self.root.children.values())
        while stack:
            n = stack.pop()
            yield n
            stack.extend(n.children.values())

    def _owns(self, group: int, page: int) -> int:
        return sum(1 for n in self._nodes() if n.pages[group] == page)
