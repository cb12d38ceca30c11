"""Page bookkeeping of the sliding-window K/V pool
(python/minisgl/kvcache/swa_window.py:46-113, python/minisgl/engine/engine.py:484-523).

Layers that only attend to the last ``window`` positions keep their K/V in a pool of their own.
A request's pages in that pool are taken as its positions are written and handed back as soon as
every position on them has left the window of the next query, so a request holds about
``window / page_size + 2`` pages however long its context is (plus the pages of a prefill chunk
while that chunk runs). The pool is sized for that bound times the number of request slots, so
an allocation cannot fail and admission does not have to look at it.

A page can have several holders (the request that wrote it, requests admitted with a reused
prefix, windows kept for the prefix cache) and goes back to the free list with its last one.

The table lives on the host (numpy) and is mirrored on the device: every change is noted and
``flush`` sends the noted entries in one small copy on the engine's stream, ahead of the step that
needs them and behind the step that last read the old values. The engine derives the per-row
slots and the per-request block table of a step from the device copy, so plans, padding and
captured graphs need no second set of page arrays.

The reference keeps a fixed ring per request (slot = position modulo stride). Pages with a free
list give the same bound without tying the stride to the largest prefill chunk.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch


class SwaPages:
    def __init__(self, num_slots: int, max_pages_per_seq: int, num_pages: int, page_size: int, window: int,
                 device) -> None:
        self.page_size, self.window = int(page_size), int(window)
        self.dummy = int(num_pages)                       # the pool has one page more than it hands out
        self.table = np.full((num_slots, max_pages_per_seq), self.dummy, dtype=np.int32)
        self.first = np.zeros(num_slots, dtype=np.int64)  # first page index a slot still holds
        self.next = np.zeros(num_slots, dtype=np.int64)   # one past the last page index it holds
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self.device = torch.device(device)
        self.table_dev = torch.full((num_slots, max_pages_per_seq), self.dummy, dtype=torch.int32, device=self.device)
        self._dirty: Dict[int, int] = {}             # flat table index -> value (the last change of a cell wins)
        # holders of every page: the request that wrote it, requests that adopted it with a reused prefix,
        # windows kept for the prefix cache
        self.refs = np.zeros(num_pages + 1, dtype=np.int32)
        self._kept: Dict[object, tuple] = {}         # key -> (first page index, page ids, boundary)
        self.page_nbytes = 0                         # bytes of one page over all sliding layers (set by the engine)
        self.peak_in_use = 0
        self.num_pages = int(num_pages)

    @property
    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def _set(self, slot: int, page_idx: int, value: int) -> None:
        self.table[slot, page_idx] = value
        self._dirty[slot * self.table.shape[1] + page_idx] = value

    def ensure(self, slot: int, end_pos: int) -> None:
        """Pages for every position below ``end_pos`` that the slot does not hold yet."""
        need = (int(end_pos) + self.page_size - 1) // self.page_size
        nxt = int(self.next[slot])
        if need <= nxt:
            return
        if len(self._free) < need - nxt:
            raise RuntimeError(f"sliding-window pool exhausted: {need - nxt} pages wanted, {len(self._free)} free "
                               f"(the pool is sized for window + chunk per request)")
        for p in range(nxt, need):
            page = self._free.pop()
            self.refs[page] = 1
            self._set(slot, p, page)
        self.next[slot] = need
        self.peak_in_use = max(self.peak_in_use, self.in_use)

    def trim(self, slot: int, next_query_pos: int) -> None:
        """Hand back pages whose positions are all outside the window of a query at
        ``next_query_pos`` (it sees positions ``> next_query_pos - window``) and of every later one."""
        keep_from = max(0, (int(next_query_pos) - self.window + 1)) // self.page_size
        f = int(self.first[slot])
        stop = min(keep_from, int(self.next[slot]))
        for p in range(f, stop):
            self._unref(int(self.table[slot, p]))
            self._set(slot, p, self.dummy)
        if stop > f:
            self.first[slot] = stop

    def release(self, slot: int) -> None:
        for p in range(int(self.first[slot]), int(self.next[slot])):
            self._unref(int(self.table[slot, p]))
            self._set(slot, p, self.dummy)
        self.first[slot] = self.next[slot] = 0

    def _unref(self, page: int) -> None:
        self.refs[page] -= 1
        if self.refs[page] == 0:
            self._free.append(page)

    # ---- windows kept for prefix reuse (the interface of the recurrent-state snapshots) ----
    def slot_nbytes(self) -> int:
        """Bytes one kept window pins in the pool."""
        return ((self.window + self.page_size - 1) // self.page_size) * max(self.page_nbytes, 1)

    @property
    def num_snapshots(self) -> int:
        return len(self._kept)

    def snapshot(self, slot: int, key, host: bool = False, end: int = 0) -> None:
        """Keep the pages that hold the window below the page-aligned boundary ``end`` of ``slot``'s
        sequence: a later request that reuses the prefix ``[0, end)`` reads them in place
        (python/minisgl/kvcache/swa_window.py:46-113 copies the window out of a ring instead)."""
        lo, hi = max(0, end - self.window) // self.page_size, end // self.page_size
        pages = self.table[slot, lo:hi].copy()
        if hi > int(self.next[slot]) or lo < int(self.first[slot]) or (pages == self.dummy).any():
            return                                    # the window is not all there any more: nothing to keep
        self.refs[pages] += 1
        self._kept[key] = (lo, pages, int(end))

    def restore(self, slot: int, key) -> bool:
        """A request admitted with the prefix ``[0, end)`` of a kept window takes the window's pages
        into its own table (shared, read only: it writes from position ``end`` on, i.e. into later pages)."""
        kept = self._kept.get(key)
        if kept is None:
            return False
        lo, pages, _end = kept
        self.release(slot)
        for i, page in enumerate(pages.tolist()):
            self.refs[page] += 1
            self._set(slot, lo + i, int(page))
        self.first[slot], self.next[slot] = lo, lo + len(pages)
        return True

    def drop_snapshot(self, key) -> None:
        kept = self._kept.pop(key, None)
        if kept is not None:
            for page in kept[1].tolist():
                self._unref(int(page))

    def flush(self) -> None:
        """Send the noted entries to the device copy (on the current stream)."""
        if not self._dirty:
            return
        idx = torch.tensor(list(self._dirty.keys()), dtype=torch.int64)
        val = torch.tensor(list(self._dirty.values()), dtype=torch.int32)
        self._dirty = {}
        if self.device.type == "cuda":
            idx = idx.pin_memory().to(self.device, non_blocking=True)
            val = val.pin_memory().to(self.device, non_blocking=True)
        self.table_dev.view(-1)[idx] = val

    def check(self) -> None:
        count = np.zeros(self.num_pages + 1, dtype=np.int64)
        for v in self.table.reshape(-1):
            if v != self.dummy:
                count[int(v)] += 1
        for _lo, pages, _end in self._kept.values():
            count[pages] += 1
        assert (count[: self.num_pages] == self.refs[: self.num_pages]).all(), "sliding-window page holders are off"
        free = set(self._free)
        assert len(free) == len(self._free), "a sliding-window page is free twice"
        assert all((self.refs[p] == 0) == (p in free) for p in range(self.num_pages)), "sliding-window pages leaked"
