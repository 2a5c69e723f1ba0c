from .manager import CacheManager
from .pages import RELEASED, CacheGroup, GroupSpec, PagePool, PoolExhausted, SlotPool
from .storage import CacheStorage

__all__ = ["CacheGroup", "CacheManager", "CacheStorage", "GroupSpec", "PagePool", "PoolExhausted", "RELEASED", "SlotPool"]
