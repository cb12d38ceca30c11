"""Pinned host arena for weights that live off the device
(python/minisgl/weights/pinned_arena.py:1-327, python/minisgl/weights/chunk_plan.py).

Two steps, so that a plan that cannot fit fails before anything is page-locked:

* ``reserve(name, shape, dtype)`` is integer arithmetic only: every region gets an aligned offset
  inside a chunk; a region never straddles two chunks (each chunk is one page-locked allocation with
  its own address range), a region larger than the chunk size gets a chunk of its own;
* ``attach()`` checks the total against what the host can spare (``host_capacity.check_pinned``),
  makes one page-locked allocation per chunk and hands out typed views. After that the arena is
  frozen: weights are written once and read for the life of the process, so there is no free list.

``put(name, tensor)`` keeps the one-call form for callers that have the tensor in hand: it is
reserve + attach of a private chunk + copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

ALIGN = 512                      # every region starts on a 512-byte boundary of its chunk
DEFAULT_CHUNK = 2 << 30          # bytes per page-locked allocation


def _round_up(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


@dataclass
class Region:
    name: str
    chunk: int
    offset: int
    nbytes: int
    shape: Tuple[int, ...]
    dtype: torch.dtype


class ChunkPlan:
    """Where every named region goes; no memory behind it."""

    def __init__(self, chunk_bytes: int = DEFAULT_CHUNK) -> None:
        self.chunk_bytes = int(chunk_bytes)
        self.regions: Dict[str, Region] = {}
        self.chunk_sizes: List[int] = []          # bytes used per chunk
        self._sealed = False                      # the open chunk already has memory: start a new one

    def reserve(self, name: str, shape, dtype: torch.dtype) -> Region:
        if name in self.regions:
            raise KeyError(f"region {name!r} is already reserved")
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        need = _round_up(max(nbytes, 1))
        if (need > self.chunk_bytes or not self.chunk_sizes or self._sealed
                or self.chunk_sizes[-1] + need > self.chunk_bytes):
            self.chunk_sizes.append(0)            # open a new chunk (an oversized region has it to itself)
            self._sealed = False
        idx = len(self.chunk_sizes) - 1
        region = Region(name, idx, self.chunk_sizes[idx], nbytes, tuple(int(s) for s in shape), dtype)
        self.chunk_sizes[idx] += need
        self.regions[name] = region
        return region

    def seal(self) -> None:
        """The chunks reserved so far got their memory: later regions go to new chunks."""
        self._sealed = True

    @property
    def total_bytes(self) -> int:
        return sum(self.chunk_sizes)


class PinnedArena:
    def __init__(self, pin: bool = True, chunk_bytes: int = DEFAULT_CHUNK) -> None:
        self.pin = pin and torch.cuda.is_available()
        self.plan = ChunkPlan(chunk_bytes)
        self._chunks: List[torch.Tensor] = []
        self._attached = 0                        # chunks of the plan that have memory
        self.tensors: Dict[str, torch.Tensor] = {}
        self.frozen = False

    # ---- two-step form ----
    def reserve(self, name: str, shape, dtype: torch.dtype) -> Region:
        if self.frozen:
            raise RuntimeError("the arena is frozen: every region has to be reserved before attach()")
        return self.plan.reserve(name, shape, dtype)

    def attach(self, freeze: bool = True, check_capacity: bool = True) -> None:
        """Page-lock the chunks reserved so far and build the views."""
        todo = self.plan.chunk_sizes[self._attached:]
        if check_capacity and self.pin and todo:
            from .host_capacity import check_pinned

            check_pinned(sum(todo))
        for size in todo:
            self._chunks.append(torch.empty(max(size, ALIGN), dtype=torch.uint8, pin_memory=self.pin))
        self._attached = len(self.plan.chunk_sizes)
        self.plan.seal()
        for name, r in self.plan.regions.items():
            if name in self.tensors:
                continue
            flat = self._chunks[r.chunk][r.offset:r.offset + r.nbytes]
            self.tensors[name] = flat.view(r.dtype).view(r.shape)
        self.frozen = self.frozen or freeze

    # ---- one-call form ----
    def put(self, name: str, t: torch.Tensor) -> torch.Tensor:
        src = t.detach()
        self.plan.reserve(name, tuple(src.shape), src.dtype)
        self.attach(freeze=False)
        host = self.tensors[name]
        host.copy_(src)
        return host

    def get(self, name: str) -> torch.Tensor:
        return self.tensors[name]

    @property
    def nbytes(self) -> int:
        return sum(r.nbytes for r in self.plan.regions.values())

    @property
    def num_chunks(self) -> int:
        return len(self._chunks)
