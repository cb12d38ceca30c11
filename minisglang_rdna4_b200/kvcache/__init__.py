"""Paged KV pools and prefix caches."""
from __future__ import annotations

from .base import BaseCacheHandle, BaseKVCachePool, BasePrefixCache, SizeInfo
from .naive_cache import NaivePrefixCache
from .radix_cache import RadixPrefixCache, SnapshotRadixCache
from .mha_pool import MHAKVCache


def create_prefix_cache(kind: str, page_size: int) -> BasePrefixCache:
    """``radix`` or ``naive`` (python/minisgl/kvcache/__init__.py:60-101)."""
    if kind == "radix":
        return RadixPrefixCache(page_size)
    if kind == "radix_snapshot":
        return SnapshotRadixCache(page_size)
    if kind == "naive":
        return NaivePrefixCache(page_size)
    raise ValueError(f"unknown cache type {kind!r}")


__all__ = [
    "BaseCacheHandle",
    "BaseKVCachePool",
    "BasePrefixCache",
    "SizeInfo",
    "NaivePrefixCache",
    "RadixPrefixCache",
    "SnapshotRadixCache",
    "MHAKVCache",
    "create_prefix_cache",
]
