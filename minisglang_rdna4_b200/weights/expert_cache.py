"""Segmented-LRU residency cache for experts (python/minisgl/weights/expert_cache.py:147).

Keys enter a probationary segment; a second hit promotes them to the protected segment, whose
overflow is demoted back to probation. Victims always come from the cold end of probation, so a
burst of one-off experts cannot flush the experts that are hit every step. Values are device
slot indices."""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Set, Tuple


class SLRUCache:
    def __init__(self, capacity: int, protected_fraction: float = 0.8) -> None:
        if capacity < 1:
            raise ValueError("capacity must be positive")
        self.capacity = capacity
        self.protected_cap = max(0, min(capacity - 1, int(capacity * protected_fraction)))
        self.probation: "OrderedDict[int, int]" = OrderedDict()
        self.protected: "OrderedDict[int, int]" = OrderedDict()
        self.free_slots: List[int] = list(range(capacity - 1, -1, -1))
        self.hits = self.misses = self.evictions = 0

    def __contains__(self, key: int) -> bool:
        return key in self.probation or key in self.protected

    def __len__(self) -> int:
        return len(self.probation) + len(self.protected)

    def slot_of(self, key: int) -> Optional[int]:
        if key in self.protected:
            return self.protected[key]
        return self.probation.get(key)

    def touch(self, key: int) -> Optional[int]:
        """Record a use. Returns the slot on a hit, None on a miss."""
        if key in self.protected:
            self.protected.move_to_end(key)
            self.hits += 1
            return self.protected[key]
        if key in self.probation:
            slot = self.probation.pop(key)
            self.hits += 1
            if self.protected_cap > 0:
                self.protected[key] = slot
                while len(self.protected) > self.protected_cap:
                    old, old_slot = self.protected.popitem(last=False)
                    self.probation[old] = old_slot
            else:
                self.probation[key] = slot
            return slot
        self.misses += 1
        return None

    def admit(self, key: int, pinned: Iterable[int] = ()) -> Tuple[int, Optional[int]]:
        """Give ``key`` a slot, evicting if needed (never one of ``pinned``). Returns
        ``(slot, evicted key or None)``."""
        assert key not in self
        evicted = None
        if self.free_slots:
            slot = self.free_slots.pop()
        else:
            keep: Set[int] = set(pinned)
            victim = next((k for k in self.probation if k not in keep), None)
            if victim is None:
                victim = next((k for k in self.protected if k not in keep), None)
                if victim is None:
                    raise RuntimeError("every resident expert is needed by the current step")
                slot = self.protected.pop(victim)
            else:
                slot = self.probation.pop(victim)
            evicted = victim
            self.evictions += 1
        self.probation[key] = slot
        return slot, evicted

    def stats(self) -> Dict[str, float]:
        total = self.hits + self.misses
        return {"hits": self.hits, "misses": self.misses, "evictions": self.evictions,
                "hit_rate": self.hits / total if total else 0.0, "resident": len(self)}
