"""Radix / prefix cache: the C++ core (``native``) and the routing facades built on it."""

from .config import CacheConfig, Modality
from .encoding import (ImageSegment, encode_chunk_hash_atoms_u64, encode_eagle_bigram_atoms, encode_image_hash_atom_sha256,
                       encode_prompt_to_atoms, encode_text_atoms_int32, page_align)
from .hybrid import HybridCache, HybridCacheConfig
from .multimodal import MultimodalCache, MultiPatternCache, NestedCache
from .native import (CacheError, CacheEventKind, HybridMatchResult, HybridPrefixCache, MambaSlot, MatchResult, PrefixCache,
                     StorageBackend, Tier, file_storage_backend, hash64, in_memory_storage_backend)
from .paired import PairedCache, PairedCacheConfig, PairedMatchResult


def __getattr__(name: str):
    if name in ("CacheCapacityError", "CacheUsageError", "CacheInvariantError"):
        from . import native

        return getattr(native, name)
    raise AttributeError(name)


__all__ = ["CacheConfig", "Modality", "ImageSegment", "page_align", "encode_text_atoms_int32", "encode_eagle_bigram_atoms",
           "encode_chunk_hash_atoms_u64", "encode_image_hash_atom_sha256", "encode_prompt_to_atoms", "HybridCache",
           "HybridCacheConfig", "MultimodalCache", "MultiPatternCache", "NestedCache", "PairedCache", "PairedCacheConfig",
           "PairedMatchResult", "PrefixCache", "HybridPrefixCache", "MatchResult", "HybridMatchResult", "MambaSlot", "Tier",
           "CacheEventKind", "CacheError", "StorageBackend", "in_memory_storage_backend", "file_storage_backend", "hash64",
           "CacheCapacityError", "CacheUsageError", "CacheInvariantError"]
