from .cache import KVView, RunCache, SequenceCache
from .pages import PAGE_TOKENS, CacheError, FreeList, PageTable

__all__ = ["KVView", "RunCache", "SequenceCache", "PAGE_TOKENS", "CacheError", "FreeList", "PageTable"]
