from .needs import CacheNeeds, KVNeed, StateNeed
from .paged import Cache, EntryView
from .slots import CacheFull, FreeList

__all__ = ["Cache", "EntryView", "CacheNeeds", "KVNeed", "StateNeed", "CacheFull", "FreeList"]
