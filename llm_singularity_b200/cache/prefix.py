"""RadixPrefixCache: requests leave their full pages behind for later prompts, the prompt's
pages as soon as the prompt has run, the rest when the request ends.

A tree keyed by page-sized chunks of token ids; a node owns one page per cache
group (the keys and values of that chunk after the path above it).  A new prompt
walks the tree and adopts the pages of its longest cached prefix instead of
recomputing them.  Only whole pages are shared, and a match never covers the
last prompt token, so there is always something to run and logits to return.
Nodes no live request uses are evictable, leaves first, least recently used
first; the scheduler evicts when the pools run short.

The reference's ``PrefixCache`` is a map from whole prompts to page lists with a
linear longest-prefix scan (core/src/memory.cpp:46-83); it hands out a donor's
partial last page, never releases a reference it took and never calls
``evict_lru`` outside its test, so donated pages never return
(core/src/scheduler.cpp:43-65,90-102).  This tree is the block-aligned radix
cache its design notes intended.
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Sequence, Tuple

from .manager import CacheManager


class _Node:
    __slots__ = ("key", "pages", "children", "parent", "users", "last_used")

    def __init__(self, key, pages, parent):
        self.key: Tuple[int, ...] = key
        self.pages: Tuple[int, ...] = pages          # one page id per cache group
        self.children: Dict[Tuple[int, ...], "_Node"] = {}
        self.parent: Optional["_Node"] = parent
        self.users = 0                               # live requests whose prefix runs through here
        self.last_used = 0


class RadixPrefixCache:
    def __init__(self, cache: CacheManager):
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
