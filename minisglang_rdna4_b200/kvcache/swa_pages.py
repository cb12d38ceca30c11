"""Page bookkeeping of the sliding-window K/V pool
(python/minisgl/kvcache/swa_window.py:46-113, python/minisgl/engine/engine.py:484-523).

Layers that only attend to the last ``window`` positions keep their K/V in a pool of their own.
A request's pages in that pool are taken as its positions are written and handed back as soon as
every position on them has left the window of the next query, so a request holds about
``window / page_size + 2`` pages however long its context is (plus the pages of a prefill chunk
while that chunk runs). The pool is sized for that bound times the number of request slots, so
an allocation cannot fail and admission does not have to look at it.

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
            self._set(slot, p, self._free.pop())
        self.next[slot] = need
        self.peak_in_use = max(self.peak_in_use, self.in_use)

    def trim(self, slot: int, next_query_pos: int) -> None:
        """Hand back pages whose positions are all outside the window of a query at
        ``next_query_pos`` (it sees positions ``> next_query_pos - window``) and of every later one."""
        keep_from = max(0, (int(next_query_pos) - self.window + 1)) // self.page_size
        f = int(self.first[slot])
        stop = min(keep_from, int(self.next[slot]))
        for p in range(f, stop):
            self._free.append(int(self.table[slot, p]))
            self._set(slot, p, self.dummy)
        if stop > f:
            self.first[slot] = stop

    def release(self, slot: int) -> None:
        for p in range(int(self.first[slot]), int(self.next[slot])):
            self._free.append(int(self.table[slot, p]))
            self._set(slot, p, self.dummy)
        self.first[slot] = self.next[slot] = 0

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
        held = [int(v) for v in self.table.reshape(-1) if v != self.dummy]
        assert len(held) == len(set(held)), "a sliding-window page is mapped twice"
        assert len(held) + len(self._free) == self.num_pages, "sliding-window pages leaked"
