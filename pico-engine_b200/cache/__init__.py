"""The cache: sequence slots, paged keys and values per group of layers, per-sequence state."""
from .needs import CacheNeeds, KVNeed
from .pages import CacheFull, CacheStateError, FreeList
from .cache import Cache, KVGroup, PAGE, pages_for

__all__ = ["CacheNeeds", "KVNeed", "CacheFull", "CacheStateError", "FreeList", "Cache", "KVGroup", "PAGE", "pages_for"]
