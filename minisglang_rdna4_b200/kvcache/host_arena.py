"""Pinned host arena of fixed-size frames for state snapshots
(python/minisgl/kvcache/host_arena.py:132-274).

A snapshot of a request's recurrent state (all layers' convolution tails and state matrices) has
one size for the life of the engine, and snapshots come and go with the prefix cache. So the arena
is one page-locked slab cut into identical frames with a FIFO free list: a frame that was just
released is the last to be handed out again. A released frame may still be the source or target of
a copy in flight; ``release`` takes the event recorded behind that copy and ``alloc`` waits on it.
No decision here depends on whether an event has completed (no ``query()``): two tensor-parallel
ranks make the same allocations in the same order whatever their timing.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import torch

ALIGN = 256


def _round_up(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


@dataclass
class Component:
    name: str
    offset: int                 # bytes from the start of a frame
    shape: Tuple[int, ...]
    dtype: torch.dtype
    nbytes: int


class FrameLayout:
    """Byte layout of one frame: named components, each on a 256-byte boundary. Pure arithmetic."""

    def __init__(self, components: Sequence[Tuple[str, Sequence[int], torch.dtype]]) -> None:
        self.components: List[Component] = []
        off = 0
        for name, shape, dtype in components:
            numel = 1
            for s in shape:
                numel *= int(s)
            nbytes = numel * torch.empty((), dtype=dtype).element_size()
            self.components.append(Component(name, off, tuple(int(s) for s in shape), dtype, nbytes))
            off += _round_up(nbytes)
        self.frame_bytes = max(off, ALIGN)

    def frames_in(self, budget_bytes: int) -> int:
        return int(budget_bytes) // self.frame_bytes


class PinnedFrameArena:
    def __init__(self, layout: FrameLayout, num_frames: int, pin: bool = True) -> None:
        if num_frames <= 0:
            raise ValueError("a frame arena needs at least one frame")
        self.layout = layout
        self.num_frames = int(num_frames)
        self.pinned = bool(pin and torch.cuda.is_available())
        self._slab = torch.empty(self.num_frames * layout.frame_bytes, dtype=torch.uint8, pin_memory=self.pinned)
        self._free: Deque[int] = deque(range(self.num_frames))
        self._busy: Dict[int, object] = {}       # frame -> event behind its last copy
        self._held = set()

    @property
    def nbytes(self) -> int:
        return int(self._slab.numel())

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> Optional[int]:
        """A frame nobody holds, or ``None`` when all are held. Waits for the frame's last copy."""
        if not self._free:
            return None
        idx = self._free.popleft()
        ev = self._busy.pop(idx, None)
        if ev is not None:
            ev.synchronize()
        self._held.add(idx)
        return idx

    def release(self, idx: int, event=None) -> None:
        """Idempotent: a snapshot can be dropped from several paths."""
        if idx not in self._held:
            return
        self._held.discard(idx)
        if event is not None:
            self._busy[idx] = event
        self._free.append(idx)

    def views(self, idx: int) -> Dict[str, torch.Tensor]:
        base = idx * self.layout.frame_bytes
        out = {}
        for c in self.layout.components:
            flat = self._slab[base + c.offset: base + c.offset + c.nbytes]
            out[c.name] = flat.view(c.dtype).view(c.shape)
        return out

    def __del__(self) -> None:  # interpreter shutdown may already have torn the module down
        try:
            self._busy.clear()
        except Exception:
            pass
