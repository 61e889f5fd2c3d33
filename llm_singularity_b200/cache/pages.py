"""PagePool: the free list and reference counts of one group's cache pages.

A page id addresses the same slot in the key pool and the value pool of every
layer of its group, as in the reference (models/llama/llama_model.h:56-69), whose
``BlockPool`` is a bare stack of indices (core/src/memory.cpp:5-38) that never
notices a page freed twice.  This pool counts references (a page shared through
the prefix cache is held by several owners) and raises on a double free, a free
of a page never handed out, or a retain of a free page.

The counts live in the host memory layer (``csrc/host_memory.cpp``); this class is
a view of one group's pool there, or of a pool of its own when made from a size.
"""
from __future__ import annotations

from typing import Optional

from . import native


class PageError(RuntimeError):
    pass


class _Handle:
    """Owner of one native ``Memory`` object."""

    def __init__(self, page_size, max_requests, max_pages, windows, num_pages):
        self.lib = native.lib()
        self.ptr = self.lib.lsbm_create(page_size, max_requests, max_pages, len(windows),
                                        native.ints(windows), native.ints(num_pages))
        if not self.ptr:
            raise ValueError("the memory layer needs positive sizes "
                             f"(page_size {page_size}, slots {max_requests}, table {max_pages}, "
                             f"pages {list(num_pages)})")

    def __del__(self):
        if getattr(self, "ptr", None):
            self.lib.lsbm_destroy(self.ptr)
            self.ptr = None

    def error(self) -> PageError:
        return PageError(self.lib.lsbm_last_error(self.ptr).decode())


class PagePool:
    def __init__(self, num_pages: int, _handle: Optional[_Handle] = None, _group: int = 0):
        if _handle is None:
            if num_pages <= 0:
                raise ValueError(f"a page pool needs at least one page, got {num_pages}")
            _handle = _Handle(1, 1, 1, [-1], [num_pages])
        self._h, self._g = _handle, _group
        self.num_pages = num_pages

    @property
    def num_free(self) -> int:
        return self._h.lib.lsbm_pool_num_free(self._h.ptr, self._g)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.num_free

    def allocate(self) -> Optional[int]:
        """A free page with one reference, or ``None`` if the pool is empty."""
        p = self._h.lib.lsbm_pool_allocate(self._h.ptr, self._g)
        return None if p < 0 else p

    def retain(self, page: int) -> None:
        if self._h.lib.lsbm_pool_retain(self._h.ptr, self._g, page) == native.ERR:
            raise self._h.error()

    def release(self, page: int) -> bool:
        """Drop one reference; returns True if the page went back to the free list."""
        rc = self._h.lib.lsbm_pool_release(self._h.ptr, self._g, page)
        if rc == native.ERR:
            raise self._h.error()
        return rc == 1

    def refcount(self, page: int) -> int:
        rc = self._h.lib.lsbm_pool_refcount(self._h.ptr, self._g, page)
        if rc == native.ERR:
            raise self._h.error()
        return rc

    def check_invariants(self) -> None:
        if self._h.lib.lsbm_pool_check(self._h.ptr, self._g) == native.ERR:
            raise self._h.error()
