"""Host-side allocator of fixed-size pages.  A page is held by exactly one
owner or lies in the free list; giving back a page that is not held is an
error, so that no page is lost, held twice or freed twice."""
from __future__ import annotations

from typing import List

PAGE_SIZE = 64   # tokens per page; the unit in which a cache is sized


class CacheFull(RuntimeError):
    """No free page (or slot) is left for what a step needs."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = int(n_pages)
        self._free: List[int] = list(range(self.n_pages - 1, -1, -1))   # pop() hands out 0 first
        self._held = [False] * self.n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_pages} pages of the cache are in use")
        p = self._free.pop()
        self._held[p] = True
        return p

    def give_back(self, page: int) -> None:
        if not 0 <= page < self.n_pages:
            raise ValueError(f"page {page} does not belong to this pool of {self.n_pages}")
        if not self._held[page]:
            raise ValueError(f"page {page} is given back but is not held (freed twice?)")
        self._held[page] = False
        self._free.append(page)

    def check(self) -> None:
        """Every page is either free or held, never both, none missing."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is in the free list twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise AssertionError(f"page {p} is {'held and free' if self._held[p] else 'lost'}")
