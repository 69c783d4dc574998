from .manager import (CacheError, CacheFull, CacheManager, CacheView, FixedState, PagedKV,
                      PagePool)

__all__ = ["CacheError", "CacheFull", "CacheManager", "CacheView", "FixedState", "PagedKV",
           "PagePool"]
