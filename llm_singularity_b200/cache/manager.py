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

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheSpec, KVCacheView, StateView      # noqa: F401  (views re-exported)
from . import native
from .pages import PageError, PagePool, _Handle

NO_PAGE = -1


class _Group:
    """One group's Python face: its pool and its host table are views into the memory layer."""

    def __init__(self, handle: _Handle, index: int, window: Optional[int], num_pages: int,
                 slots: int, max_pages: int, page_size: int):
        self.index = index
        self.window = window
        self.page_size = page_size
        self.pool = PagePool(num_pages, _handle=handle, _group=index)
        self.cache_ids: List[int] = []
        ptr = handle.lib.lsbm_table(handle.ptr, index)
        self.table = np.ctypeslib.as_array(ptr, shape=(slots, max_pages))   # host mirror (no copy)
        self.dev_table: Optional[torch.Tensor] = None


_NO_INTS = np.empty(0, dtype=np.int32)


class CacheManager:
    def __init__(self, cache_specs: Sequence[object], page_size: int, num_pages,
                 max_requests: int, max_pages_per_request: int, rt=None):
        """``cache_specs[i]`` is what cache id ``i`` holds (a ``CacheSpec`` or None);
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
        self._store: Dict[int, object] = {}            # cache id -> what its spec allocated
        self._slots: Dict[Hashable, int] = {}          # request id -> slot

        windows: List[Optional[int]] = []              # one entry per group, in order of first use
        members: List[List[int]] = []
        for cid, cs in enumerate(self._specs):
            if cs is None:
                continue
            if not isinstance(cs, CacheSpec):
                raise TypeError(f"cache {cid}: {cs!r} is not a CacheSpec")
            if cs.paged:                               # caches with one release rule share a group
                if cs.window not in windows:
                    windows.append(cs.window)
                    members.append([])
                g = windows.index(cs.window)
                members[g].append(cid)
                self._group_of[cid] = g
        sizes = [num_pages[w] if isinstance(num_pages, dict) else num_pages for w in windows]
        if any(n <= 0 for n in sizes):
            raise ValueError(f"a page pool needs at least one page, got {sizes}")
        self._h = _Handle(page_size, max_requests, max_pages_per_request,
                          [-1 if w is None else w for w in windows], sizes)
        self._lib, self._ptr = self._h.lib, self._h.ptr
        for g, (w, n) in enumerate(zip(windows, sizes)):
            grp = _Group(self._h, g, w, n, max_requests, max_pages_per_request, page_size)
            grp.cache_ids = members[g]
            self.groups.append(grp)
        self._page_buf = (ctypes.c_int * max_pages_per_request)()
        self._update_buf: Dict[int, np.ndarray] = {}
        if rt is not None:
            self._allocate_device(rt)

    # ------------------------------------------------------------------ device
    def _allocate_device(self, rt) -> None:
        for g in self.groups:
            g.dev_table = torch.full(g.table.shape, NO_PAGE, dtype=torch.int32, device=rt.device)
        for cid, cs in enumerate(self._specs):
            if cs is not None:
                n = self.groups[self._group_of[cid]].pool.num_pages if cs.paged else None
                self._store[cid] = cs.allocate(rt, self.page_size, n, self.max_requests)

    def bytes_per_page(self, group: int) -> int:
        """Bytes one page id stands for, over all layers of the group (keys and values)."""
        esize = 4 if self.rt is None else torch.empty((), dtype=self.rt.dtype).element_size()
        return sum(self._specs[c].bytes_per_page(self.page_size, esize)
                   for c in self.groups[group].cache_ids)

    # ---------------------------------------------------------------- requests
    def _fail(self, request=None) -> PageError:
        msg = self._lib.lsbm_last_error(self._ptr).decode()
        return PageError(msg if request is None else f"request {request!r}: {msg}")

    def has(self, request: Hashable) -> bool:
        return request in self._slots

    def open(self, request: Hashable) -> Optional[int]:
        """Give ``request`` a slot (block-table row and state row); None if all are taken."""
        if request in self._slots:
            raise KeyError(f"request {request!r} is already open")
        slot = self._lib.lsbm_open(self._ptr)
        if slot < 0:
            return None
        self._slots[request] = slot
        self._reset(slot)
        return slot

    def bind(self, request: Hashable, slot: int) -> None:
        """``slot`` was opened inside the memory layer (by the scheduler, which lives there too)
        and now belongs to ``request``."""
        if request in self._slots:
            raise KeyError(f"request {request!r} is already open")
        self._slots[request] = slot
        self._reset(slot)

    def _reset(self, slot: int) -> None:
        for cid, store in self._store.items():
            self._specs[cid].reset(store, slot)

    def unbind(self, request: Hashable) -> None:
        """The memory layer has closed the request's slot already (see :meth:`bind`)."""
        del self._slots[request]

    def slot(self, request: Hashable) -> int:
        return self._slots[request]

    def length(self, request: Hashable) -> int:
        return self._lib.lsbm_length(self._ptr, self._slots[request])

    def pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def pages_needed(self, request: Hashable, new_length: int) -> int:
        """Pages each group must still hand out to cover ``new_length`` tokens."""
        return max(0, self.pages_for(new_length) - self._lib.lsbm_num_pages(self._ptr, self._slots[request]))

    def free_pages(self) -> int:
        """Pages free in the tightest group."""
        return self._lib.lsbm_free_pages(self._ptr)

    def reserve(self, request: Hashable, new_length: int) -> bool:
        """Cover positions ``[0, new_length)`` with pages in every group, or change nothing."""
        rc = self._lib.lsbm_reserve(self._ptr, self._slots[request], new_length)
        if rc == native.ERR:
            raise self._fail(request)
        return rc == 1

    def commit(self, request: Hashable, new_length: int) -> None:
        """The request now holds ``new_length`` tokens; give back pages a window has passed."""
        if self._lib.lsbm_commit(self._ptr, self._slots[request], new_length) == native.ERR:
            raise self._fail(request)

    def close(self, request: Hashable) -> None:
        """The request is over: every page it holds and its slot go back."""
        slot = self._slots.pop(request)
        if self._lib.lsbm_close(self._ptr, slot) == native.ERR:
            raise self._fail(request)

    def adopt(self, request: Hashable, pages_per_group: Sequence[Sequence[int]], length: int) -> None:
        """Start a fresh request on pages that already hold its first ``length`` tokens
        (shared through the prefix cache); takes one reference on each."""
        n = length // self.page_size
        if len(pages_per_group) != len(self.groups) or any(len(p) != n for p in pages_per_group):
            raise PageError("adopt: page list does not match the length")
        flat = [p for pages in pages_per_group for p in pages]
        if self._lib.lsbm_adopt(self._ptr, self._slots[request], native.ints(flat), n, length) == native.ERR:
            raise self._fail()

    def pages_of(self, request: Hashable, group: int = 0) -> List[int]:
        n = self._lib.lsbm_pages_of(self._ptr, self._slots[request], group, self._page_buf, self.max_pages)
        if n == native.ERR:
            raise self._fail(request)
        return self._page_buf[:n]

    def live_requests(self) -> List[Hashable]:
        return list(self._slots)

    # ------------------------------------------------------------------ tables
    def take_updates(self, group: int) -> List[Tuple[int, int]]:
        """Block-table cells changed since the last call, as (flat index, value)."""
        n = self._lib.lsbm_num_updates(self._ptr, group)
        if n == native.ERR:
            raise self._fail()
        if n == 0:
            return []
        buf = (ctypes.c_int * (2 * n))()
        if self._lib.lsbm_take_updates(self._ptr, group, buf, n) == native.ERR:
            raise self._fail()
        flat = buf[:]
        return list(zip(flat[0::2], flat[1::2]))

    def take_update_arrays(self, group: int) -> Tuple[np.ndarray, np.ndarray]:
        """The same as two int32 arrays (cells, values) with one entry per changed cell, its last
        value; the arrays are the manager's own and hold until the next call for the group."""
        n = self._lib.lsbm_num_updates(self._ptr, group)
        if n == native.ERR:
            raise self._fail()
        if n == 0:
            return _NO_INTS, _NO_INTS
        buf = self._update_buf.get(group)
        if buf is None or buf.shape[1] < n:
            buf = self._update_buf[group] = np.empty((2, max(2 * n, 1024)), dtype=np.int32)
        n = self._lib.lsbm_take_updates_last(self._ptr, group, buf[0].ctypes.data, buf[1].ctypes.data, buf.shape[1])
        if n == native.ERR:
            raise self._fail()
        return buf[0, :n], buf[1, :n]

    def group_of(self, cache_id: int) -> int:
        return self._group_of[cache_id]

    def view(self, cache_id: int, ctx=None):
        cs = self._specs[cache_id]
        if cs is None:
            return None
        group = self.groups[self._group_of[cache_id]] if cs.paged else None
        return cs.view(self._store.get(cache_id), group)

    # -------------------------------------------------------------- invariants
    def check_invariants(self) -> None:
        """No page lost, none held without a reference, none freed twice, no slot lost or held
        twice; references beyond those of live requests are the prefix tree's, node by node."""
        if self._lib.lsbm_check(self._ptr) == native.ERR:
            raise self._fail()
        slots = list(self._slots.values())
        if len(set(slots)) != len(slots):
            raise PageError("a slot is held twice")
