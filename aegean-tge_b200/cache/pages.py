"""Page pool: physical pages with reference counts and a LIFO free list.

Behaviour of the reference's ``BlockTable`` (include/tge/models/block_table.hpp:21-130):
``allocate`` pops the free list and sets the count to one, a full pool is an
error, ``share`` adds a reference, ``release`` drops one and returns the page
at zero, every misuse (bad id, page not live, double release) is an error,
and a page freed last is handed out first, so tests can force reuse.
"""
from __future__ import annotations

from typing import List


class PoolExhausted(RuntimeError):
    """No free page is left."""


class PageError(RuntimeError):
    """A page id was used in a way its state does not allow."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("page pool: the number of pages must be positive")
        self._refcount: List[int] = [0] * num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # page 0 is handed out first

    @property
    def capacity(self) -> int:
        return len(self._refcount)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.capacity - self.free_count

    def allocate(self) -> int:
        if not self._free:
            raise PoolExhausted("page pool: no free page")
        page = self._free.pop()
        self._refcount[page] = 1
        return page

    def _live(self, page: int) -> None:
        if not 0 <= page < self.capacity:
            raise PageError(f"page pool: page id {page} out of range")
        if self._refcount[page] <= 0:
            raise PageError(f"page pool: page {page} is not live")

    def share(self, page: int) -> None:
        self._live(page)
        self._refcount[page] += 1

    def release(self, page: int) -> bool:
        """Drops one reference; True when the page went back to the free list."""
        self._live(page)
        self._refcount[page] -= 1
        if self._refcount[page] == 0:
            self._free.append(page)
            return True
        return False

    def refcount(self, page: int) -> int:
        if not 0 <= page < self.capacity:
            raise PageError(f"page pool: page id {page} out of range")
        return self._refcount[page]

    def check(self) -> None:
        """Every page is either free exactly once or referenced, never both."""
        seen = set()
        for page in self._free:
            if page in seen:
                raise PageError(f"page pool: page {page} is on the free list twice")
            seen.add(page)
            if self._refcount[page] != 0:
                raise PageError(f"page pool: free page {page} has references")
        for page, count in enumerate(self._refcount):
            if count < 0:
                raise PageError(f"page pool: page {page} has a negative count")
            if count == 0 and page not in seen:
                raise PageError(f"page pool: page {page} is lost (neither free nor referenced)")
