"""Paged key/value cache: bookkeeping (native) and device pools."""
from .manager import CacheError, GroupSpec, OutOfPages, PageTable

__all__ = ["CacheError", "GroupSpec", "OutOfPages", "PageTable", "CachePools"]


def __getattr__(name):
    if name == "CachePools":          # needs torch and the parts; loaded on demand
        from .pools import CachePools
        return CachePools
    raise AttributeError(name)
