from .kv_cache_pool import KVCachePool
from .static_cache import StaticCache, StaticCacheError

_RADIX = ("CacheConfig", "Modality", "HybridCache", "HybridCacheConfig", "MultimodalCache", "MultiPatternCache", "NestedCache", "PairedCache",
          "PairedCacheConfig", "PairedMatchResult")


def __getattr__(name: str):
    if name in _RADIX:
        from . import radix_cache

        return getattr(radix_cache, name)
    raise AttributeError(name)


__all__ = ["KVCachePool", "StaticCache", "StaticCacheError", *_RADIX]
