from .kv_cache import PAGE, KVGroup, KVView, SequenceCache, StateGroup, StateView, pages_for
from .pages import CacheError, FreeList

__all__ = ["PAGE", "CacheError", "FreeList", "KVGroup", "KVView", "SequenceCache", "StateGroup",
           "StateView", "pages_for"]
