from .pages import PagePool
from .kinds import register_cache_kind, kind_of
from .manager import CacheManager, KVGroup

__all__ = ["PagePool", "CacheManager", "KVGroup", "register_cache_kind", "kind_of"]
