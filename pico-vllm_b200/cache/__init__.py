from .pages import PagePool
from .manager import CacheManager, KVGroup

__all__ = ["PagePool", "CacheManager", "KVGroup"]
