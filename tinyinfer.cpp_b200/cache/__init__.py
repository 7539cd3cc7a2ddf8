"""Paged cache with per-request block tables, window release and fixed-size state slots."""
from .manager import CacheManager, PagedKVView, RELEASED, StateView
from .pages import IdPool, OutOfPages

__all__ = ["CacheManager", "IdPool", "OutOfPages", "PagedKVView", "RELEASED", "StateView"]
