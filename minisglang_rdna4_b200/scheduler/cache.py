"""Page allocator + prefix-cache bookkeeping for one rank
(python/minisgl/scheduler/cache.py:17-194).

The free list and the page table live on the host: block tables are gathered per step into
the pinned staging buffer, so the device never needs the global table. A page table entry is
a page id; token slot = page * page_size + position % page_size.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..core import Req
from ..kvcache import BaseCacheHandle, BasePrefixCache, create_prefix_cache
from ..utils import cdiv


class CacheManager:
    def __init__(self, num_pages: int, page_size: int, num_slots: int, max_pages_per_seq: int,
                 cache_type: str = "radix") -> None:
        self.num_pages = num_pages
        self.page_size = page_size
        self.prefix_cache: BasePrefixCache = create_prefix_cache(cache_type, page_size)
        self._free = np.arange(num_pages - 1, -1, -1, dtype=np.int32)  # stack, top at the end
        self._n_free = num_pages
        self.page_table = np.zeros((num_slots, max_pages_per_seq), dtype=np.int32)
        self.prefix_hit_tokens = 0
        self.prefix_query_tokens = 0
        # measure-only: what an unbounded prefix cache would have reused (kvcache/ghost_oracle.py)
        self.ghost = None
        from ..kvcache.ghost_oracle import GhostPrefixOracle, oracle_enabled

        if oracle_enabled():
            self.ghost = GhostPrefixOracle(page_size)

    # ---- sizes (pages) ----
    @property
    def free_pages(self) -> int:
        return self._n_free

    @property
    def available_pages(self) -> int:
        return self._n_free + self.prefix_cache.size_info.evictable_pages

    @property
    def available_tokens(self) -> int:
        return self.available_pages * self.page_size

    @property
    def used_tokens(self) -> int:
        return (self.num_pages - self._n_free) * self.page_size

    # ---- prefix cache ----
    def match_req(self, input_ids: torch.Tensor):
        """Match all but the last prompt token so that at least one token is always computed
        (python/minisgl/scheduler/cache.py:39)."""
        n = int(input_ids.numel())
        handle, pages = self.prefix_cache.match_prefix(input_ids[: max(n - 1, 0)])
        if self.ghost is not None:
            self.ghost.observe(input_ids[: max(n - 1, 0)].tolist(), handle.cached_len)
        return handle, pages

    def lock(self, handle: BaseCacheHandle) -> None:
        self.prefix_cache.lock_handle(handle, unlock=False)

    def unlock(self, handle: BaseCacheHandle) -> None:
        self.prefix_cache.lock_handle(handle, unlock=True)

    # ---- pages ----
    def _take(self, n: int) -> np.ndarray:
        if n > self._n_free:
            need = n - self._n_free
            freed = self.prefix_cache.evict(need).numpy()
            self._give(freed)
        if n > self._n_free:
            raise RuntimeError(f"out of KV pages: want {n}, have {self._n_free}")
        out = self._free[self._n_free - n : self._n_free][::-1].copy()
        self._n_free -= n
        return out

    def _give(self, pages: np.ndarray) -> None:
        n = int(pages.size)
        if n == 0:
            return
        assert self._n_free + n <= self.num_pages, "page freed twice"
        self._free[self._n_free : self._n_free + n] = pages
        self._n_free += n

    def set_prefix_pages(self, slot: int, pages: torch.Tensor) -> None:
        n = int(pages.numel())
        if n:
            self.page_table[slot, :n] = pages.numpy()

    def allocate_for(self, req: Req, upto_len: Optional[int] = None) -> None:
        """Make sure pages exist for token positions ``[cached_len, upto_len)``."""
        ps = self.page_size
        upto = req.device_len if upto_len is None else upto_len
        first = cdiv(req.cached_len, ps)
        last = cdiv(upto, ps)
        if last > first:
            self.page_table[req.table_idx, first:last] = self._take(last - first)

    def free_tail(self, slot: int, keep_len: int, old_len: int) -> None:
        """Release pages that only held positions ``>= keep_len`` (speculative rollback)."""
        ps = self.page_size
        first, last = cdiv(keep_len, ps), cdiv(old_len, ps)
        if last > first:
            self._give(self.page_table[slot, first:last].copy())

    def slots_of(self, slot: int, start: int, end: int) -> np.ndarray:
        pos = np.arange(start, end, dtype=np.int64)
        return (self.page_table[slot, pos // self.page_size].astype(np.int64) * self.page_size
                + pos % self.page_size).astype(np.int32)

    def finish_req(self, req: Req, allocated_len: int, insert: bool = True, snapshots=None) -> list:
        """Return a finished request's pages: insert the page-aligned prefix of what was
        computed into the prefix cache, free pages that duplicate already-cached ones, free
        the unaligned tail, unlock the matched handle
        (python/minisgl/scheduler/cache.py:91-127)."""
        ps = self.page_size
        slot = req.table_idx
        handle = req.cache_handle
        n_alloc_pages = cdiv(allocated_len, ps)
        pages = self.page_table[slot, :n_alloc_pages].copy()
        valid_len = req.cached_len  # tokens whose KV is in the pool
        ids = req.input_ids[:valid_len]
        if not (insert and req.sampling_params.cache_output):
            ids = ids[: min(valid_len, req.prompt_len)]
        old_prefix_pages = handle.cached_len // ps
        # a cache that retains nothing (naive) takes ownership of no page
        keep_pages = len(ids) // ps if self.prefix_cache.retains else old_prefix_pages
        if keep_pages > old_prefix_pages:
            already = self.prefix_cache.insert_prefix(ids[: keep_pages * ps], torch.from_numpy(pages[:keep_pages]))
            already_pages = already // ps
            # pages between the handle's prefix and `already` duplicate cached content
            if already_pages > old_prefix_pages:
                self._give(pages[old_prefix_pages:already_pages])
        else:
            keep_pages = old_prefix_pages
        if n_alloc_pages > keep_pages:
            self._give(pages[keep_pages:n_alloc_pages])
        # recurrent models: state snapshots taken while the request ran become reusable prefix
        # boundaries; the ids of those that found no place in the cache go back to the caller
        unused = []
        attach = getattr(self.prefix_cache, "attach_snapshot", None)
        for length, key in (snapshots or ()):
            if attach is None or length > keep_pages * ps or not attach(ids, int(length), key):
                unused.append(key)
        self.unlock(handle)
        return unused

    def check_integrity(self) -> None:
        self.prefix_cache.check_integrity()
        info = self.prefix_cache.size_info
        free = set(self._free[: self._n_free].tolist())
        assert len(free) == self._n_free, "duplicate page in the free list"
        assert self._n_free + info.total_pages <= self.num_pages
