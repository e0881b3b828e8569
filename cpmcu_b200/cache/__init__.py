from .allocator import CacheFull, FreeList, HandleError
from .cache import Cache, CacheGroup, Lane, PAGE_TOKENS, pages_for

__all__ = ["Cache", "CacheGroup", "Lane", "CacheFull", "HandleError", "FreeList", "PAGE_TOKENS", "pages_for"]
