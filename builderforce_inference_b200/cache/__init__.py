from .cache import KVView, RunCache, SequenceCache, needs_of
from .pages import PAGE_TOKENS, CacheError, FreeList, PageTable
from .plan import CachePlan, kv_bytes_per_token, plan_cache, served_context, state_bytes_per_slot

__all__ = ["KVView", "RunCache", "SequenceCache", "needs_of", "PAGE_TOKENS", "CacheError", "FreeList", "PageTable",
           "CachePlan", "kv_bytes_per_token", "plan_cache", "served_context", "state_bytes_per_slot"]
