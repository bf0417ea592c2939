"""Bookkeeping of cache pages: which are free, which are held, by how many.

Pure host code.  The allocation order is mischief/lgml's: the lowest free page
first (``P:take``, ``lua/lgml/kvpool.lua:102-116``); pages carry reference
counts (``P:ref/unref``, ``:165-198``) so that a page can later be shared
between requests, though the engine today holds each page once.
"""
from __future__ import annotations

import heapq
from typing import List


class PoolFull(RuntimeError):
    """No free page left (mischief/lgml: "kv pool full", ``lua/lgml/transformer.lua:971``)."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages))
        heapq.heapify(self._free)
        self._refs = [0] * n_pages
        self.taken_total = 0  # pages handed out since the start: shows reuse

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise PoolFull(f"kv pool full: {self.n_held} of {self.n_pages} pages in use")
        p = heapq.heappop(self._free)
        assert self._refs[p] == 0, f"page {p} was free but held"
        self._refs[p] = 1
        self.taken_total += 1
        return p

    def ref(self, page: int) -> None:
        if not (0 <= page < self.n_pages) or self._refs[page] <= 0:
            raise ValueError(f"page {page} is not held")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        if not (0 <= page < self.n_pages):
            raise ValueError(f"page {page} is outside the pool of {self.n_pages}")
        if self._refs[page] <= 0:
            raise ValueError(f"page {page} freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            heapq.heappush(self._free, page)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def check(self) -> None:
        """Every page is either free once or held, never both, never lost."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.n_pages):
            if (self._refs[p] == 0) != (p in set(free)):
                raise AssertionError(f"page {p}: refcount {self._refs[p]} disagrees with the free list")
