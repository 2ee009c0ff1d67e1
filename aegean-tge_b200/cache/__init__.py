"""Paged cache and per-request state slots."""
from .manager import NO_PAGE, CacheManager, PageGroup
from .pages import PageError, PagePool, PoolExhausted

__all__ = ["NO_PAGE", "CacheManager", "PageGroup", "PageError", "PagePool", "PoolExhausted"]
