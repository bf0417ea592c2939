"""Bookkeeping of cache pages: which are free, which are held, by how many.

Pure host code.  The allocation order is mischief/lgml's: the lowest free page
first (``P:take``, ``lua/lgml/kvpool.lua:102-116``); pages carry reference
counts (``P:ref/unref``, ``:165-198``) so that a page can be shared between
requests.  A page may carry a *key* (of the tokens it and the pages before it
hold, ``P:publish`` ``:217``): another request with the same tokens finds it by
``lookup`` (``:261``) and shares it, and when its last holder lets go it stays
*cached*, neither free nor held, until the pool needs it: ``take`` uses the free
pages first and then the cached one that was let go longest ago
(``P:evict`` ``:139-160``).
"""
from __future__ import annotations

import heapq
from collections import OrderedDict
from typing import Dict, List, Optional


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
        self._key_of: Dict[int, bytes] = {}                 # page -> its key
        self._page_of: Dict[bytes, int] = {}                # key -> the page that holds those tokens
        self._cached: "OrderedDict[int, None]" = OrderedDict()   # keyed pages nobody holds, oldest first
        self.taken_total = 0  # pages handed out since the start: shows reuse
        self.shared_total = 0  # pages found by their key and shared
        self.evicted_total = 0  # cached pages that lost their key to a request in need

    @property
    def n_free(self) -> int:
        """Pages a request can still get: the free ones and the cached ones."""
        return len(self._free) + len(self._cached)

    @property
    def n_cached(self) -> int:
        return len(self._cached)

    @property
    def n_held(self) -> int:
        return self.n_pages - self.n_free

    def take(self) -> int:
        if self._free:
            p = heapq.heappop(self._free)
        elif self._cached:
            p, _ = self._cached.popitem(last=False)          # the one let go longest ago
            del self._page_of[self._key_of.pop(p)]
            self.evicted_total += 1
        else:
            raise PoolFull(f"kv pool full: {self.n_held} of {self.n_pages} pages in use")
        assert self._refs[p] == 0, f"page {p} was free but held"
        self._refs[p] = 1
        self.taken_total += 1
        return p

    # ---- keyed pages -----------------------------------------------------------------------
    def publish(self, page: int, key: bytes) -> bool:
        """Give a held page its key.  False (and no change) when another page already has
        that key or this page another key."""
        if not (0 <= page < self.n_pages) or self._refs[page] <= 0:
            raise ValueError(f"page {page} is not held")
        if key in self._page_of or page in self._key_of:
            return self._page_of.get(key) == page
        self._key_of[page] = key
        self._page_of[key] = page
        return True

    def lookup(self, key: bytes) -> Optional[int]:
        return self._page_of.get(key)

    def share(self, page: int) -> None:
        """One more holder of a keyed page, held or cached."""
        if page in self._cached:
            del self._cached[page]
            self._refs[page] = 1
        elif 0 <= page < self.n_pages and self._refs[page] > 0 and page in self._key_of:
            self._refs[page] += 1
        else:
            raise ValueError(f"page {page} is neither cached nor a held page with a key")
        self.shared_total += 1

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
            if page in self._key_of:
                self._cached[page] = None                   # stays findable until the pool needs it
            else:
                heapq.heappush(self._free, page)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def check(self) -> None:
        """Every page is either free once or held, never both, never lost."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        if free & set(self._cached):
            raise AssertionError("a page is both free and cached")
        for p in range(self.n_pages):
            if (self._refs[p] == 0) != (p in free or p in self._cached):
                raise AssertionError(f"page {p}: refcount {self._refs[p]} disagrees with the free and cached lists")
            if p in self._cached and p not in self._key_of:
                raise AssertionError(f"page {p} is cached without a key")
            if p in free and p in self._key_of:
                raise AssertionError(f"page {p} is free but still has a key")
        if len(self._key_of) != len(self._page_of) or any(self._page_of.get(k) != p for p, k in self._key_of.items()):
            raise AssertionError("the keys of pages and the pages of keys disagree")
