"""Row-chunked all-reduce under the compute of the next chunk
(python/minisgl/layers/tp_overlap.py:276-417).

A row-parallel block of a prefill step (the experts of a MoE layer under tensor parallelism)
produces partial sums of ``[rows, hidden]`` that the next fused add + norm would all-reduce in one
piece, after the block is done. Rows are independent, so the block can run chunk by chunk: while
the experts work on chunk ``i + 1`` the partial sums of chunk ``i`` are already being reduced on a
second stream. The block then returns finished rows and the following norm does not reduce.

Off unless ``MSGL_TP_OVERLAP=1``, and only for steps of at least ``MSGL_TP_OVERLAP_MIN_ROWS`` rows:
small steps are latency bound and take the fused all-reduce + norm kernel. On CPU ranks (gloo)
the chunks simply run one after the other; the arithmetic is the same.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..env import ENV
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info

_side_stream: Optional["torch.cuda.Stream"] = None


def applies(rows: int) -> bool:
    return bool(ENV.TP_OVERLAP.value) and get_tp_info().size > 1 and rows >= ENV.TP_OVERLAP_MIN_ROWS.value


def chunked_all_reduce(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, chunks: int = 0) -> torch.Tensor:
    """``all_reduce(fn(x))`` computed over row chunks; ``fn`` maps ``[r, ...]`` rows to ``[r, H]``
    partial sums and must treat rows independently."""
    global _side_stream
    rows = x.shape[0]
    chunks = chunks or max(2, min(ENV.TP_OVERLAP_CHUNKS.value, rows // 128 or 1))
    step = -(-rows // chunks)
    step = -(-step // 128) * 128 if rows >= 256 else step       # whole 128-row tiles for the grouped GEMMs
    comm = get_comm()
    parts = []
    if not x.is_cuda:
        for lo in range(0, rows, step):
            parts.append(comm.all_reduce(fn(x[lo:lo + step])))
        return torch.cat(parts)
    if _side_stream is None:
        _side_stream = torch.cuda.Stream(x.device)
    main = torch.cuda.current_stream()
    for lo in range(0, rows, step):
        y = fn(x[lo:lo + step])
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(_side_stream):
            _side_stream.wait_event(ready)
            y = comm.all_reduce(y)
            y.record_stream(_side_stream)
        parts.append(y)
    main.wait_stream(_side_stream)
    return torch.cat(parts)
