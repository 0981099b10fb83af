from .manager import PAGE_TOKENS, CacheGroup, CacheManager, LayerCache, Sequence, pages_for
from .pool import CacheFull, IndexPool

__all__ = ["PAGE_TOKENS", "CacheGroup", "CacheManager", "LayerCache", "Sequence", "pages_for", "CacheFull",
           "IndexPool"]
