"""Expert parallelism across data-parallel replicas (DP+EP).

Every replica routes its own tokens; experts are sharded ``[rank * E/ep, (rank+1) * E/ep)``.
Baseline data plane (what the reference does, python/minisgl/layers/moe.py:1244-1311): gather
every replica's token rows and routing, run the local experts over all rows with non-local
experts masked out, sum the partial outputs over the replicas and keep the own rows. All
replicas must issue the same collectives with the same shapes, so the scheduler agrees on a
common padded token count per step (``scheduler/ep.py``) and stores it in ``common_tokens``.
The fused path (``csrc/ep_a2a.cu`` when present) replaces gather + reduce with P2P stores of
only the rows each expert owner needs and of the weighted results back.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class EPContext:
    def __init__(self, group: Optional[dist.ProcessGroup], rank: int, size: int) -> None:
        self.group, self.rank, self.size = group, rank, size
        self.common_tokens: Optional[int] = None
        self.calls = 0

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.size * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def dispatch_compute_combine(self, moe, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor
                                 ) -> torch.Tensor:
        n_local = x.shape[0]
        n = self.common_tokens
        if n is None:
            # eager step without a scheduler agreement: agree here (one small collective)
            cnt = torch.tensor([n_local], dtype=torch.int64, device=x.device)
            dist.all_reduce(cnt, op=dist.ReduceOp.MAX, group=self.group)
            n = int(cnt.item())
        if n < n_local:
            raise RuntimeError(f"expert-parallel step agreed on {n} rows but this replica has {n_local}")
        pad = n - n_local
        if pad:
            x = torch.cat([x, x.new_zeros((pad, x.shape[1]))])
            topk_w = torch.cat([topk_w, topk_w.new_zeros((pad, topk_w.shape[1]))])
            topk_ids = torch.cat([topk_ids, topk_ids.new_full((pad, topk_ids.shape[1]), -1)])
        xs, ws, ids = self._gather(x), self._gather(topk_w), self._gather(topk_ids)
        y = moe.local_experts(xs, ws, ids)
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        self.calls += 1
        return y[self.rank * n : self.rank * n + n_local]
