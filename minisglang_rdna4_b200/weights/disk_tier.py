"""Disk tier of the expert weights (python/minisgl/weights/stream_tier.py:135, ckpt_read.py:353,
row_table.py:233): experts that the pinned host arena cannot hold live in one flat file per tensor
family, one fixed-size record per (layer, expert), and are read into a caller-provided (pinned)
buffer on demand. Records are padded to 4096 bytes so that a read can bypass the page cache
(``O_DIRECT``) when the buffer is aligned; without alignment the reader falls back to buffered
``preadv``. The reference's io_uring submission queue is replaced by plain positional reads on a
small thread pool: one expert is a few MB, so the queue depth that matters is the number of
experts in flight, not of 4 KB blocks."""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Tuple

import numpy as np
import torch

_ALIGN = 4096


def _padded(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


class ExpertFile:
    """``[layers][experts]`` records of one tensor family."""

    def __init__(self, path: str, layers: int, experts: int, shape: Tuple[int, ...], dtype: torch.dtype) -> None:
        self.path, self.layers, self.experts = path, layers, experts
        self.shape, self.dtype = tuple(shape), dtype
        self.record_bytes = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.stride = _padded(self.record_bytes)
        self._fd = -1
        self._direct = False

    def offset(self, layer: int, expert: int) -> int:
        if not (0 <= layer < self.layers and 0 <= expert < self.experts):
            raise IndexError(f"expert ({layer}, {expert}) outside the file's {self.layers} x {self.experts} table")
        return (layer * self.experts + expert) * self.stride

    # ------------------------------------------------------------------ writing (bake time)
    def create(self) -> None:
        with open(self.path, "wb") as fh:
            fh.truncate(self.layers * self.experts * self.stride)

    def write(self, layer: int, expert: int, t: torch.Tensor) -> None:
        if tuple(t.shape) != self.shape or t.dtype != self.dtype:
            raise ValueError(f"record is {self.shape} {self.dtype}, got {tuple(t.shape)} {t.dtype}")
        raw = t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()
        with open(self.path, "r+b") as fh:
            fh.seek(self.offset(layer, expert))
            fh.write(raw)

    # ------------------------------------------------------------------ reading (serve time)
    def open(self, direct: bool = True) -> None:
        flags = os.O_RDONLY
        self._direct = False
        if direct and hasattr(os, "O_DIRECT"):
            try:
                self._fd = os.open(self.path, flags | os.O_DIRECT)
                self._direct = True
                return
            except OSError:
                pass
        self._fd = os.open(self.path, flags)

    def close(self) -> None:
        if self._fd >= 0:
            os.close(self._fd)
            self._fd = -1

    def read_into(self, layer: int, expert: int, out: torch.Tensor) -> None:
        """``out``: CPU tensor of the record's shape and dtype (pinned for an async upload)."""
        if self._fd < 0:
            self.open()
        if tuple(out.shape) != self.shape or out.dtype != self.dtype or not out.is_contiguous():
            raise ValueError("read_into wants a contiguous tensor of the record's shape and dtype")
        view = out.view(torch.uint8).reshape(-1).numpy()
        off = self.offset(layer, expert)
        aligned = self._direct and view.ctypes.data % _ALIGN == 0 and self.record_bytes % _ALIGN == 0
        if aligned:
            got = os.preadv(self._fd, [memoryview(view)], off)
        else:
            if self._direct:   # O_DIRECT needs an aligned destination: bounce through one
                bounce = np.empty(self.stride + _ALIGN, dtype=np.uint8)
                shift = (-bounce.ctypes.data) % _ALIGN
                buf = bounce[shift:shift + self.stride]
                got = os.preadv(self._fd, [memoryview(buf)], off)
                view[:] = buf[:self.record_bytes]
                got = min(got, self.record_bytes)
            else:
                got = os.preadv(self._fd, [memoryview(view)], off)
        if got < self.record_bytes:
            raise IOError(f"short read of expert ({layer}, {expert}): {got} of {self.record_bytes} bytes")


class DiskExpertTier:
    """Several families (e.g. ``w13`` and ``w2``) read together, a few experts at a time."""

    def __init__(self, files: Dict[str, ExpertFile], workers: int = 4) -> None:
        self.files = files
        self._pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="expert-read")
        self.bytes_read = 0

    def fetch(self, layer: int, experts: List[int], out: Dict[str, torch.Tensor]) -> None:
        """``out[family][i]`` receives expert ``experts[i]``; returns when all reads are done."""
        jobs = []
        for name, f in self.files.items():
            for i, e in enumerate(experts):
                jobs.append(self._pool.submit(f.read_into, layer, e, out[name][i]))
                self.bytes_read += f.record_bytes
        for j in jobs:
            j.result()

    def close(self) -> None:
        self._pool.shutdown(wait=True)
        for f in self.files.values():
            f.close()
