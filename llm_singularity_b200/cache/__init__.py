"""Cache: page pools, block tables, state slots, prefix sharing."""
from .manager import NO_PAGE, CacheManager, KVCacheView, StateView
from .pages import PageError, PagePool

__all__ = ["NO_PAGE", "CacheManager", "KVCacheView", "StateView", "PageError", "PagePool"]
