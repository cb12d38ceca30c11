"""Tensor-parallel communicator façade.

Layers call ``get_comm().all_reduce / all_gather / fused_allreduce_add_rmsnorm``. The object
holds a chain of implementations and the last registered one that accepts the message wins
(the reference uses the same plugin order Torch → PyNCCL → CustomAR,
python/minisgl/distributed/impl.py:71-78):

* ``TorchCollectives``: ``torch.distributed`` on NCCL (GPU) or gloo (CPU ranks). This is the
  baseline data plane and the health fallback.
* ``SymmetricCollectives`` (``parallel/symm.py``): hand-written kernels over NVLink peer
  memory that fuse the all-reduce with the residual add and the next RMSNorm.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from .info import get_tp_info


class TorchCollectives:
    name = "torch"

    def __init__(self, group: Optional[dist.ProcessGroup] = None) -> None:
        self.group = group

    def accepts(self, x: torch.Tensor) -> bool:
        return True

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.group)
        return x

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        size = dist.get_world_size(self.group)
        out = torch.empty((size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        size = dist.get_world_size(self.group)
        out = torch.empty((x.shape[0] // size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out


class Communicator:
    def __init__(self) -> None:
        self.impls: List[object] = []
        self.calls = {"all_reduce": 0, "all_gather": 0, "fused_ar_norm": 0}
        # set per forward pass by the model: True only for passes in which every row-parallel
        # output feeds a fused add + norm (dense layers, no hidden-state capture)
        self.row_shard_ok = False
        # set per forward pass by the model: every row-parallel output of this pass ends in a fused
        # add + norm and the pass is a plain decode step on one GPU (see layers/linear.py)
        self.split_k_ok = False
        self._rs_impl = None

    @property
    def size(self) -> int:
        return get_tp_info().size

    def register(self, impl) -> None:
        self.impls.append(impl)

    def _pick(self, x: torch.Tensor, method: str):
        for impl in reversed(self.impls):
            if hasattr(impl, method) and impl.accepts(x):
                return impl
        raise RuntimeError(f"no collective implementation registered for {method}")

    # ---- prefill path: GEMM -> reduce-scatter -> add + norm -> all-gather -> GEMM ----
    def rs_begin(self, rows: int, hidden: int, dtype):
        """A plan for pushing a row-parallel GEMM's partial rows to their owner ranks, or None
        when this forward pass keeps the all-reduce formulation. The decision is the same at
        every fused site of a pass (same rows, same hidden): the residual stream is sharded by
        rows between those sites and must not meet the all-reduce formulation half-way."""
        if self.size == 1 or not self.row_shard_ok:
            return None
        for impl in reversed(self.impls):
            fn = getattr(impl, "rs_begin", None)
            if fn is not None:
                plan = fn(rows, hidden, dtype)
                if plan is not None:
                    plan_impl = impl
                    self._rs_impl = plan_impl
                    self.calls["fused_rs_ag"] = self.calls.get("fused_rs_ag", 0) + 1
                    return plan
        return None

    def rs_gemm_args(self, plan, a_ready=None):
        return self._rs_impl.row_shard.gemm_args(plan, a_ready)

    def rs_finish(self, plan, residual, weight, eps, quant=False, plus_one=False):
        return self._rs_impl.row_shard.finish(plan, residual, weight, eps, quant, plus_one)

    def wait_ready(self, ready) -> None:
        self._rs_impl.wait_ready(ready)

    def vocab_argmax(self, local_logits: torch.Tensor, length: int, start: int):
        """Fused shard arg-max + pair exchange when a peer-memory implementation is registered;
        None tells the caller to use the all-gather formulation."""
        if self.size == 1 or not local_logits.is_cuda:
            return None
        for impl in reversed(self.impls):
            fn = getattr(impl, "vocab_argmax", None)
            if fn is not None:
                out = fn(local_logits, length, start)
                if out is not None:
                    self.calls["vocab_argmax"] = self.calls.get("vocab_argmax", 0) + 1
                    return out
        return None

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        self.calls["all_reduce"] += 1
        return self._pick(x, "all_reduce").all_reduce(x)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        self.calls["all_gather"] += 1
        return self._pick(x, "all_gather").all_gather(x)

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        return self._pick(x, "reduce_scatter").reduce_scatter(x)

    def fused_allreduce_add_rmsnorm(self, x: torch.Tensor, residual: Optional[torch.Tensor],
                                    weight: torch.Tensor, eps: float, quant: bool = False):
        """``residual += all_reduce(x)``; returns ``rms_norm(residual)`` (or its per-token e4m3
        pair when ``quant``). With one rank, or when no fused kernel accepts the message, this
        is the unfused sequence all_reduce → add+norm."""
        if self.size > 1:
            for impl in reversed(self.impls):
                if hasattr(impl, "fused_allreduce_add_rmsnorm") and impl.accepts(x):
                    self.calls["fused_ar_norm"] += 1
                    return impl.fused_allreduce_add_rmsnorm(x, residual, weight, eps, quant)
            x = self.all_reduce(x)
        if residual is None:
            raise ValueError("fused_allreduce_add_rmsnorm needs a residual stream")
        if quant:
            return ops.rms_norm_quant(x, weight, eps, residual)
        return ops.rms_norm_add(x, residual, weight, eps)


_COMM = Communicator()


def get_comm() -> Communicator:
    return _COMM


def reset_comm() -> Communicator:
    global _COMM
    _COMM = Communicator()
    return _COMM
