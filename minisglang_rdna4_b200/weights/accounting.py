"""Device-memory ledger (python/minisgl/weights/accounting.py:152): who asked for how much, so
that the boot log can say where the GPU's memory went and an out-of-memory error can name the
largest holders instead of a bare allocator message."""
from __future__ import annotations

from typing import Dict, List, Tuple


class MemoryLedger:
    def __init__(self, capacity_bytes: int = 0) -> None:
        self.capacity = int(capacity_bytes)
        self._entries: Dict[str, int] = {}

    def add(self, name: str, nbytes: int) -> None:
        self._entries[name] = self._entries.get(name, 0) + int(nbytes)

    def release(self, name: str, nbytes: int = -1) -> None:
        have = self._entries.get(name, 0)
        left = 0 if nbytes < 0 else max(0, have - int(nbytes))
        if left:
            self._entries[name] = left
        else:
            self._entries.pop(name, None)

    @property
    def total(self) -> int:
        return sum(self._entries.values())

    def entries(self) -> List[Tuple[str, int]]:
        return sorted(self._entries.items(), key=lambda kv: -kv[1])

    def headroom(self) -> int:
        return self.capacity - self.total if self.capacity else 0

    def would_fit(self, nbytes: int) -> bool:
        return not self.capacity or self.total + int(nbytes) <= self.capacity

    def report(self) -> str:
        gib = 1 << 30
        parts = [f"{name} {n / gib:.2f} GiB" for name, n in self.entries()]
        tail = f" of {self.capacity / gib:.1f} GiB" if self.capacity else ""
        return f"device memory: {self.total / gib:.2f} GiB accounted{tail} (" + ", ".join(parts) + ")"
