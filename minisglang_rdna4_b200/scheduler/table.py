"""Request-slot allocator: a slot is one row of the page table and of the token pool
(python/minisgl/scheduler/table.py:4-21)."""
from __future__ import annotations

from typing import List


class TableManager:
    def __init__(self, max_running: int) -> None:
        self.max_running = max_running
        self._free: List[int] = list(range(max_running - 1, -1, -1))

    @property
    def available_size(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        return self._free.pop()

    def free(self, slot: int) -> None:
        assert 0 <= slot < self.max_running and slot not in self._free
        self._free.append(slot)
