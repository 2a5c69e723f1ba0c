from .manager import CacheGroup, CacheManager
from .pages import RELEASED, GroupSpec, PoolExhausted
from .storage import CacheStorage

__all__ = ["CacheGroup", "CacheManager", "CacheStorage", "GroupSpec", "PoolExhausted", "RELEASED"]
