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

import ctypes
from typing import List, Sequence, Tuple

from . import native
from .manager import CacheManager
from .pages import PageError


class NodeRef:
    """A node of the tree (the tree itself lives in the host memory layer)."""

    __slots__ = ("id", "_tree")

    def __init__(self, node_id: int, tree: "RadixPrefixCache"):
        self.id = node_id
        self._tree = tree

    @property
    def users(self) -> int:
        """Live requests whose prefix runs through this node."""
        return self._tree._int(self._tree._lib.lsbp_node_users(self._tree._ptr, self.id))

    @property
    def pages(self) -> Tuple[int, ...]:
        """One page id per cache group."""
        t = self._tree
        n = t._int(t._lib.lsbp_node_pages(t._ptr, self.id, t._group_buf))
        return tuple(t._group_buf[:n])

    def __eq__(self, other):
        return isinstance(other, NodeRef) and other.id == self.id and other._tree is self._tree

    def __hash__(self):
        return hash(self.id)

    def __repr__(self):
        return f"NodeRef({self.id})"


class RadixPrefixCache:
    def __init__(self, cache: CacheManager):
        self.cache = cache
        self.page_size = cache.page_size
        self._lib, self._ptr = cache._lib, cache._ptr
        if self._lib.lsbp_enable(self._ptr) == native.ERR:
            raise ValueError(self._lib.lsbm_last_error(self._ptr).decode())
        self._group_buf = (ctypes.c_int * max(1, len(cache.groups)))()
        self._node_buf = (ctypes.c_int * cache.max_pages)()

    def _int(self, rc: int) -> int:
        if rc == native.ERR:
            raise PageError(self._lib.lsbm_last_error(self._ptr).decode())
        return rc

    def _ids(self, path: Sequence[NodeRef]):
        return native.ints([n.id for n in path])

    @property
    def num_nodes(self) -> int:
        return self._lib.lsbp_num_nodes(self._ptr)

    @property
    def hits(self) -> int:
        """Pages adopted instead of recomputed."""
        return self._lib.lsbp_hits(self._ptr)

    # ---------------------------------------------------------------- lookup
    def match(self, tokens: Sequence[int]) -> List[NodeRef]:
        """Nodes of the longest cached prefix of ``tokens`` (whole pages, never the last token)."""
        keep, ptr = native.token_array(tokens)
        n = self._int(self._lib.lsbp_match(self._ptr, ptr, len(keep), self._node_buf, self.cache.max_pages))
        return [NodeRef(i, self) for i in self._node_buf[:n]]

    def adopt(self, request, path: List[NodeRef]) -> int:
        """Start ``request`` (open, no pages yet) on the pages of ``path``; returns tokens covered."""
        if not path:
            return 0
        return self._int(self._lib.lsbp_adopt(self._ptr, self.cache.slot(request), self._ids(path), len(path)))

    def release(self, path: List[NodeRef]) -> None:
        """The request that adopted ``path`` is gone (its page references are dropped by close)."""
        self._int(self._lib.lsbp_release(self._ptr, self._ids(path), len(path)))

    def idle_on(self, path: Sequence[NodeRef]) -> int:
        """How many nodes of ``path`` no live request uses: they count among the evictable pages,
        but not for a request that is about to adopt them."""
        return self._int(self._lib.lsbp_idle_on(self._ptr, self._ids(path), len(path)))

    # ---------------------------------------------------------------- insert
    def insert(self, tokens: Sequence[int], request) -> int:
        """Keep the full pages of ``request`` (which holds ``tokens``) for later prompts.
        Call before the request is closed.  Returns the number of pages newly kept."""
        keep, ptr = native.token_array(tokens)
        return self._int(self._lib.lsbp_insert(self._ptr, ptr, len(keep), self.cache.slot(request)))

    def share(self, tokens: Sequence[int], request, held: Sequence[NodeRef]) -> List[NodeRef]:
        """Like :meth:`insert`, for a request that goes on running: the pages its ``tokens`` fill
        become visible to later prompts now (a prompt that arrives while this one still decodes
        need not recompute what they have in common).  ``held``: the nodes the request already counts
        as a user of (its adopted prefix).  Returns the further nodes whose pages are the
        request's own; it is a user of those too until :meth:`release`, so that they are not
        offered for eviction while evicting them would free nothing."""
        keep, ptr = native.token_array(tokens)
        n = self._int(self._lib.lsbp_share(self._ptr, ptr, len(keep), self.cache.slot(request),
                                           self._ids(held), len(held), self._node_buf, self.cache.max_pages))
        return [NodeRef(i, self) for i in self._node_buf[:n]]

    # -------------------------------------------------------------- eviction
    def evictable_pages(self) -> int:
        return self._lib.lsbp_evictable(self._ptr)

    def evict(self, pages_wanted: int) -> int:
        """Give back up to ``pages_wanted`` pages per group (unused leaves, least recently used
        first); returns how many were freed."""
        if pages_wanted <= 0:
            return 0
        return self._int(self._lib.lsbp_evict(self._ptr, pages_wanted))

    def check_invariants(self) -> None:
        """The counters agree with the tree (tests call this)."""
        self.cache.check_invariants()
