"""Page pool: physical pages with reference counts and a LIFO free list.

Behaviour of the reference's ``BlockTable`` (include/tge/models/block_table.hpp:21-130):
``allocate`` pops the free list and sets the count to one, a full pool is an
error, ``share`` adds a reference, ``release`` drops one and returns the page
at zero, every misuse (bad id, page not live, double release) is an error,
and a page freed last is handed out first, so tests can force reuse.

The pool itself is C++ (csrc/runtime.cpp); this class is a view of one, either
its own or one that a cache manager's group owns.
"""
from __future__ import annotations

from .. import runtime as _rt
from ..runtime import PageError, PoolExhausted  # noqa: F401  (re-exported)


class PagePool:
    def __init__(self, num_pages: int = 0, *, _borrowed=None):
        self._lib = _rt.lib()
        if _borrowed is not None:
            self._handle, self._owned = _borrowed, False
            return
        if num_pages <= 0:
            raise ValueError("page pool: the number of pages must be positive")
        self._handle, self._owned = self._lib.tge_rt_pool_create(int(num_pages)), True

    def __del__(self):
        if getattr(self, "_owned", False) and self._handle:
            self._lib.tge_rt_pool_destroy(self._handle)
            self._handle = None

    @property
    def capacity(self) -> int:
        return self._lib.tge_rt_pool_capacity(self._handle)

    @property
    def free_count(self) -> int:
        return self._lib.tge_rt_pool_free_count(self._handle)

    @property
    def used_count(self) -> int:
        return self.capacity - self.free_count

    def allocate(self) -> int:
        return _rt.check(self._lib.tge_rt_pool_allocate(self._handle))

    def share(self, page: int) -> None:
        _rt.check(self._lib.tge_rt_pool_share(self._handle, int(page)))

    def release(self, page: int) -> bool:
        """Drops one reference; True when the page went back to the free list."""
        return _rt.check(self._lib.tge_rt_pool_release(self._handle, int(page))) == 1

    def refcount(self, page: int) -> int:
        return _rt.check(self._lib.tge_rt_pool_refcount(self._handle, int(page)))

    def check(self) -> None:
        """Every page is either free exactly once or referenced, never both."""
        _rt.check(self._lib.tge_rt_pool_check(self._handle))
