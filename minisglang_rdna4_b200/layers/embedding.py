"""Vocabulary-parallel embedding and LM head
(python/minisgl/layers/embedding.py:83-242).

Each rank owns ``ceil(V / tp)`` consecutive vocabulary rows. The embedding looks up the ids
it owns (others give zero rows) and all-reduces; the head computes ``[rows, V/tp]`` logits,
all-gathers them and restores vocabulary order. For greedy decoding the head can instead
return the arg-max id directly, reducing (value, id) pairs across ranks with ties going to
the lowest rank, which is the lowest id.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..utils import cdiv
from .base import BaseOP


class VocabParallelEmbedding(BaseOP):
    def __init__(self, vocab: int, hidden: int, dtype, device) -> None:
        tp = get_tp_info()
        self._vocab = vocab
        self._per_rank = cdiv(vocab, tp.size)
        self._start = tp.rank * self._per_rank
        self._len = max(0, min(self._per_rank, vocab - self._start))
        self._tp = tp
        self.weight = torch.empty((self._per_rank, hidden), dtype=dtype, device=device)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self._tp.size == 1:
            return ops.embedding(ids, self.weight)
        y = ops.embedding(ids, self.weight, self._start, self._len)
        return get_comm().all_reduce(y)

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        w = torch.randn(self.weight.shape, generator=gen, device=gen.device, dtype=torch.float32) * std
        self.weight = w.to(self.weight.device, self.weight.dtype)


class ParallelLMHead(BaseOP):
    def __init__(self, vocab: int, hidden: int, dtype, device,
                 tied: Optional[VocabParallelEmbedding] = None) -> None:
        tp = get_tp_info()
        self._vocab = vocab
        self._per_rank = cdiv(vocab, tp.size)
        self._start = tp.rank * self._per_rank
        self._len = max(0, min(self._per_rank, vocab - self._start))
        self._tp = tp
        self._tied = tied
        if tied is None:
            self.weight = torch.empty((self._per_rank, hidden), dtype=dtype, device=device)

    @property
    def _w(self) -> torch.Tensor:
        return self._tied.weight if self._tied is not None else self.weight

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 logits of this rank's vocabulary shard ``[rows, ceil(V / tp)]`` (columns past the
        shard's length are padding)."""
        return ops.gemm(x, self._w, None, torch.float32)

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        """Shard logits → full-vocabulary logits ``[rows, V]`` on every rank."""
        if self._tp.size == 1:
            return local[:, : self._vocab]
        rows = local.shape[0]
        gathered = get_comm().all_gather(local.contiguous())            # [tp * rows, V/tp]
        full = gathered.view(self._tp.size, rows, self._per_rank).permute(1, 0, 2).reshape(rows, -1)
        return full[:, : self._vocab]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 logits ``[rows, V]``."""
        return self.gather(self.forward_local(x))

    def argmax_from_local(self, local: torch.Tensor) -> torch.Tensor:
        """Greedy token ids from shard logits without materialising the full vocabulary anywhere:
        every rank reduces its shard to (max, index) and only those pairs are exchanged
        (vocabulary-parallel arg-max, python/minisgl/layers/embedding.py:196-242). Ties go to the
        lowest index, as a full-row arg-max would."""
        logits = local[:, : self._len]
        if self._tp.size == 1:
            return ops.argmax(logits)
        fused = get_comm().vocab_argmax(local, self._len, self._start)
        if fused is not None:
            return fused
        if self._len > 0:
            val, idx = logits.max(dim=-1)
        else:  # a rank whose shard is entirely past the vocabulary
            val = torch.full((local.shape[0],), float("-inf"), device=local.device)
            idx = torch.zeros(local.shape[0], dtype=torch.long, device=local.device)
        pair = torch.stack([val, (idx + self._start).float()], dim=-1)   # [rows, 2]
        allp = get_comm().all_gather(pair).view(self._tp.size, -1, 2)
        best = allp[..., 0].argmax(dim=0)   # first maximum = lowest rank = lowest index on ties
        return allp[best, torch.arange(allp.shape[1], device=local.device), 1].to(torch.int32)

    def forward_argmax(self, x: torch.Tensor) -> torch.Tensor:
        return self.argmax_from_local(self.forward_local(x))

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        if self._tied is None:
            w = torch.randn(self.weight.shape, generator=gen, device=gen.device, dtype=torch.float32) * std
            self.weight = w.to(self.weight.device, self.weight.dtype)
