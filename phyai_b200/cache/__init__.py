from .kv_cache_pool import KVCachePool
from .static_cache import StaticCache

__all__ = ["KVCachePool", "StaticCache"]
