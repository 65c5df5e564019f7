from .cache import PAGE_SIZE, Cache
from .group import CacheGroup, CacheSizing
from .paged import KVView, PagedKVGroup
from .slots import CacheError, SlotAllocator
from .state import StateGroup

__all__ = ["PAGE_SIZE", "Cache", "CacheGroup", "CacheSizing", "KVView", "PagedKVGroup", "CacheError", "SlotAllocator",
           "StateGroup"]
