from .page_pool import PagePool, OutOfPages
from .kv_cache import KVCacheManager, KVCacheStorage, bytes_per_token
from .state_slots import StateSlotManager, StateSlotStorage, OutOfSlots

__all__ = ["PagePool", "OutOfPages", "KVCacheManager", "KVCacheStorage", "bytes_per_token",
           "StateSlotManager", "StateSlotStorage", "OutOfSlots"]
