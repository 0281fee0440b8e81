from .spec import CacheSpec, FixedStateSpec, PagedKVSpec
from .page_pool import OutOfPages, PagePool, hash_block
from .state_slots import OutOfSlots, StateSlotPool
from .manager import CacheGroup, CacheManager, RequestCache

__all__ = ["CacheSpec", "FixedStateSpec", "PagedKVSpec", "OutOfPages", "PagePool", "hash_block",
           "OutOfSlots", "StateSlotPool", "CacheGroup", "CacheManager", "RequestCache"]
