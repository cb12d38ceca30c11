"""Pinned host arena holding the full set of expert weights
(python/minisgl/weights/pinned_arena.py:327). One page-locked allocation per tensor family so a
miss is a single contiguous ``cudaMemcpyAsync`` per expert and family."""
from __future__ import annotations

from typing import Dict

import torch


class PinnedArena:
    def __init__(self, pin: bool = True) -> None:
        self.pin = pin and torch.cuda.is_available()
        self.tensors: Dict[str, torch.Tensor] = {}

    def put(self, name: str, t: torch.Tensor) -> torch.Tensor:
        host = t.detach().to("cpu").contiguous()
        if self.pin:
            host = host.pin_memory()
        self.tensors[name] = host
        return host

    def get(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())
