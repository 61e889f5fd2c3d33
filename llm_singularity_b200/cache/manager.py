"""CacheManager: pages, block tables and state slots for every live request.

Layers are sorted into groups by what their mixer needs: all past keys
(``window is None``) or only the last ``window``.  Each group has its own
:class:`PagePool` and its own block table per request; a page id addresses one
slot in the key pool and the value pool of every layer of the group.  Pages are
taken before a step for the tokens that step brings, handed back when a request
ends or, in a windowed group, as soon as the window has passed them, and reused.
Mixers with per-request state of fixed size get one row per request slot
instead of pages.  The slot of a request is also its row in the block tables.

The reference keeps one group, allocates a whole prompt's pages at admission
and grows tables after sampling, silently stopping when the pool is empty so
that the next forward writes into page 0 (core/src/scheduler.cpp:20-41,225-235;
models/llama/llama_model.cpp:343,358).  Here ``reserve`` either covers the new
length in every group or changes nothing and says so.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import PagedKVSpec, StateSpec
from .pages import PageError, PagePool

NO_PAGE = -1


@dataclass
class KVCacheView:
    """What an attention call sees of its cache."""

    k_pages: torch.Tensor          # [num_pages, kv_heads, page_size, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor      # int32 [slots, max_pages]; rows picked by ctx.table_rows
    page_size: int
    window: Optional[int]
    group: int


@dataclass
class StateView:
    """What a mixer with fixed-size state sees: ``state[ctx.table_rows[r]]`` is request r's."""

    state: torch.Tensor            # [slots, *shape]


class _Group:
    def __init__(self, window: Optional[int], num_pages: int, slots: int, max_pages: int):
        self.window = window
        self.pool = PagePool(num_pages)
        self.cache_ids: List[int] = []
        self.table = np.full((slots, max_pages), NO_PAGE, dtype=np.int32)   # host mirror
        self.dev_table: Optional[torch.Tensor] = None
        self.updates: List[Tuple[int, int]] = []       # (flat index, value) not yet on device
        # per request: pages [0, first_live) have been released behind the window
        self.first_live: Dict[Hashable, int] = {}


class _Request:
    __slots__ = ("slot", "length", "num_pages")

    def __init__(self, slot: int):
        self.slot = slot
        self.length = 0
        self.num_pages = 0     # logical pages covered so far (same count in every group)


class CacheManager:
    def __init__(self, cache_specs: Sequence[object], page_size: int, num_pages,
                 max_requests: int, max_pages_per_request: int, rt=None):
        """``cache_specs[i]`` is what cache id ``i`` holds (PagedKVSpec, StateSpec or None);
        ``num_pages`` is an int (every group gets that many) or ``{window: pages}``."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_pages = max_pages_per_request
        self.rt = rt
        self.groups: List[_Group] = []
        self._group_of: Dict[int, int] = {}
        self._specs = list(cache_specs)
        self._kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._state: Dict[int, torch.Tensor] = {}
        self._requests: Dict[Hashable, _Request] = {}
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))

        by_window: Dict[Optional[int], int] = {}
        for cid, cs in enumerate(self._specs):
            if isinstance(cs, PagedKVSpec):
                if cs.window not in by_window:
                    n = num_pages[cs.window] if isinstance(num_pages, dict) else num_pages
                    by_window[cs.window] = len(self.groups)
                    self.groups.append(_Group(cs.window, n, max_requests, max_pages_per_request))
                g = by_window[cs.window]
                self.groups[g].cache_ids.append(cid)
                self._group_of[cid] = g
            elif not (cs is None or isinstance(cs, StateSpec)):
                raise TypeError(f"cache {cid}: unknown cache spec {cs!r}")
        if rt is not None:
            self._allocate_device(rt)

    # ------------------------------------------------------------------ device
    def _allocate_device(self, rt) -> None:
        for g in self.groups:
            g.dev_table = torch.full(g.table.shape, NO_PAGE, dtype=torch.int32, device=rt.device)
        for cid, cs in enumerate(self._specs):
            if isinstance(cs, PagedKVSpec):
                n = self.groups[self._group_of[cid]].pool.num_pages
                shape = (n, cs.num_kv_heads, self.page_size, cs.head_dim)
                self._kv[cid] = (torch.zeros(shape, dtype=rt.dtype, device=rt.device),
                                 torch.zeros(shape, dtype=rt.dtype, device=rt.device))
            elif isinstance(cs, StateSpec):
                self._state[cid] = torch.zeros((self.max_requests,) + tuple(cs.shape),
                                               dtype=cs.dtype, device=rt.device)

    def bytes_per_page(self, group: int) -> int:
        """Bytes one page id stands for, over all layers of the group (keys and values)."""
        esize = 4 if self.rt is None else torch.empty((), dtype=self.rt.dtype).element_size()
        return sum(2 * self._specs[c].num_kv_heads * self.page_size * self._specs[c].head_dim * esize
                   for c in self.groups[group].cache_ids)

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
        for st in self._state.values():
            st[slot].zero_()
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

    def group_of(self, cache_id: int) -> int:
        return self._group_of[cache_id]

    def view(self, cache_id: int, ctx=None):
        cs = self._specs[cache_id]
        if isinstance(cs, PagedKVSpec):
            gi = self._group_of[cache_id]
            g = self.groups[gi]
            k, v = self._kv[cache_id]
            return KVCacheView(k, v, g.dev_table, self.page_size, g.window, gi)
        if isinstance(cs, StateSpec):
            return StateView(self._state[cache_id])
        return None

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
