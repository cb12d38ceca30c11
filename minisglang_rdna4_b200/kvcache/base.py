"""Interfaces of the paged KV pool and of the prefix caches
(python/minisgl/kvcache/base.py:10,67)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import NamedTuple, Tuple

import torch


class BaseKVCachePool(ABC):
    """Storage of K and V for every layer, addressed by token slot = page * page_size + offset."""

    num_layers: int
    num_pages: int
    page_size: int

    @abstractmethod
    def k_cache(self, layer: int) -> torch.Tensor: ...

    @abstractmethod
    def v_cache(self, layer: int) -> torch.Tensor: ...

    @abstractmethod
    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer: int) -> None: ...

    @property
    @abstractmethod
    def device(self) -> torch.device: ...

    @property
    @abstractmethod
    def dtype(self) -> torch.dtype: ...


@dataclass
class BaseCacheHandle(ABC):
    cached_len: int  # tokens, a multiple of the page size


class SizeInfo(NamedTuple):
    evictable_pages: int
    protected_pages: int

    @property
    def total_pages(self) -> int:
        return self.evictable_pages + self.protected_pages


class BasePrefixCache(ABC):
    retains = True  # False for a cache that never keeps inserted pages

    @abstractmethod
    def match_prefix(self, input_ids: torch.Tensor) -> Tuple[BaseCacheHandle, torch.Tensor]:
        """Longest cached page-aligned prefix of ``input_ids``: handle plus its page ids."""

    @abstractmethod
    def lock_handle(self, handle: BaseCacheHandle, unlock: bool = False) -> None: ...

    @abstractmethod
    def insert_prefix(self, input_ids: torch.Tensor, page_ids: torch.Tensor) -> int:
        """Insert ``input_ids`` (aligned down to whole pages) backed by ``page_ids``.
        Returns how many leading tokens were already cached (their pages are duplicates
        that the caller frees)."""

    @abstractmethod
    def evict(self, num_pages: int) -> torch.Tensor:
        """Free at least ``num_pages`` unlocked pages; returns their ids."""

    @abstractmethod
    def reset(self) -> None: ...

    @property
    @abstractmethod
    def size_info(self) -> SizeInfo: ...

    @abstractmethod
    def check_integrity(self) -> None: ...
