"""PagePool: the free list and reference counts of one group's cache pages.

A page id addresses the same slot in the key pool and the value pool of every
layer of its group, as in the reference (models/llama/llama_model.h:56-69), whose
``BlockPool`` is a bare stack of indices (core/src/memory.cpp:5-38) that never
notices a page freed twice.  This pool counts references (a page shared through
the prefix cache is held by several owners) and raises on a double free, a free
of a page never handed out, or a retain of a free page.
"""
from __future__ import annotations

from typing import List, Optional


class PageError(RuntimeError):
    pass


class PagePool:
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
