"""Prefix cache that caches nothing (``--cache-type naive``;
python/minisgl/kvcache/naive_cache.py)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

from .base import BaseCacheHandle, BasePrefixCache, SizeInfo


@dataclass
class NaiveHandle(BaseCacheHandle):
    pass


class NaivePrefixCache(BasePrefixCache):
    retains = False

    def __init__(self, page_size: int) -> None:
        self.page_size = page_size
        self._empty = torch.empty(0, dtype=torch.int32)

    def match_prefix(self, input_ids: torch.Tensor) -> Tuple[NaiveHandle, torch.Tensor]:
        return NaiveHandle(0), self._empty

    def lock_handle(self, handle: BaseCacheHandle, unlock: bool = False) -> None:
        return None

    def insert_prefix(self, input_ids: torch.Tensor, page_ids: torch.Tensor) -> int:
        return 0

    def evict(self, num_pages: int) -> torch.Tensor:
        if num_pages > 0:
            raise RuntimeError("the naive prefix cache holds no evictable pages")
        return self._empty

    def reset(self) -> None:
        return None

    @property
    def size_info(self) -> SizeInfo:
        return SizeInfo(0, 0)

    def check_integrity(self) -> None:
        return None
