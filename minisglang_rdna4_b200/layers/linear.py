"""Tensor-parallel linear layers (Megatron style).

Column-parallel layers shard the output dimension, row-parallel layers shard the input
dimension and leave a partial sum that still has to be all-reduced. The all-reduce is NOT
issued here: the decoder layer hands the partial sum to the fused
all-reduce + residual-add + RMSNorm op. The reference all-reduces inside ``forward``
(python/minisgl/layers/linear.py:104-222); ``forward(..., reduce=True)`` gives that
behaviour where a caller needs a finished sum.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..parallel.comm import get_comm
from ..parallel.info import get_tp_info
from ..quant.config import QuantScheme
from ..quant.method import ActQ, LinearInput, LinearMethod, make_linear_method
from ..utils import div_even
from .base import BaseOP


class _LinearBase(BaseOP):
    """Owns the tensors its linear method declares, as attributes named like the
    checkpoint suffixes (``weight``, ``weight_scale``, ``qweight`` …)."""

    def __init__(self, n_local: int, k_local: int, dtype: torch.dtype, device,
                 scheme: Optional[QuantScheme], bias: bool) -> None:
        self._n, self._k = n_local, k_local
        self._compute_dtype = dtype
        self._method: LinearMethod = make_linear_method(scheme)
        for name, tensor in self._method.create_weights(n_local, k_local, dtype, device).items():
            setattr(self, name, tensor)
        if bias:
            self.bias = torch.empty((n_local,), dtype=dtype, device=device)

    @property
    def wants_act_quant(self) -> bool:
        return self._method.wants_act_quant

    def _post_load_self(self) -> None:
        self._method.process_after_load(self)

    def _mm(self, x: LinearInput) -> torch.Tensor:
        ready = getattr(x, "ready", None)
        if ready is not None:
            # rows that peers are still delivering: the GEMM waits per 128-row block
            from ..ops import cuda as K

            K.set_next_gemm_tp(ready.gemm_args())
            y = self._method.apply(self, x, getattr(self, "bias", None))
            if K.take_pending_gemm_tp() is not None:
                raise RuntimeError("linear method did not consume the pending all-gather arguments")
            return y
        return self._method.apply(self, x, getattr(self, "bias", None))

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        self._method.init_dummy(self, gen, std)
        if hasattr(self, "bias"):
            self.bias = torch.zeros_like(self.bias)


class ReplicatedLinear(_LinearBase):
    def __init__(self, k: int, n: int, dtype, device, scheme=None, bias: bool = False) -> None:
        super().__init__(n, k, dtype, device, scheme, bias)

    def forward(self, x: LinearInput) -> torch.Tensor:
        return self._mm(x)


class ColumnParallelLinear(_LinearBase):
    def __init__(self, k: int, n: int, dtype, device, scheme=None, bias: bool = False) -> None:
        tp = get_tp_info().size
        super().__init__(div_even(n, tp), k, dtype, device, scheme, bias)

    def forward(self, x: LinearInput) -> torch.Tensor:
        return self._mm(x)


class MergedColumnParallelLinear(_LinearBase):
    """Several column-parallel projections of the same input stored as one weight
    (gate_proj ‖ up_proj)."""

    def __init__(self, k: int, ns: Sequence[int], dtype, device, scheme=None, bias: bool = False) -> None:
        tp = get_tp_info().size
        self._parts: List[int] = [div_even(n, tp) for n in ns]
        super().__init__(sum(self._parts), k, dtype, device, scheme, bias)

    def forward(self, x: LinearInput) -> torch.Tensor:
        return self._mm(x)


class QKVParallelLinear(_LinearBase):
    """q ‖ k ‖ v with KV-head replication when there are fewer KV heads than ranks
    (python/minisgl/layers/linear.py:132-171)."""

    def __init__(self, hidden: int, head_dim: int, num_q: int, num_kv: int, dtype, device,
                 scheme=None, bias: bool = False) -> None:
        tp = get_tp_info().size
        self._q_local = div_even(num_q, tp)
        self._kv_local = div_even(num_kv, tp, allow_replicate=True)
        self._head_dim = head_dim
        n = (self._q_local + 2 * self._kv_local) * head_dim
        super().__init__(n, hidden, dtype, device, scheme, bias)

    def forward(self, x: LinearInput) -> torch.Tensor:
        return self._mm(x)


class RowParallelLinear(_LinearBase):
    def __init__(self, k: int, n: int, dtype, device, scheme=None, bias: bool = False) -> None:
        tp = get_tp_info()
        super().__init__(n, div_even(k, tp.size), dtype, device, scheme, bias)
        self._tp_rank = tp.rank

    def forward(self, x: LinearInput, reduce: bool = False):
        # the bias must be added once, not once per rank
        bias = getattr(self, "bias", None) if self._tp_rank == 0 else None
        comm = get_comm()
        if not reduce and comm.size > 1:
            rows = x.shape[0] if len(x.shape) == 2 else 0
            plan = comm.rs_begin(rows, self._n, self._compute_dtype) if rows else None
            if plan is not None:
                # GEMM -> reduce-scatter: the epilogue stores every partial row block into the
                # memory of the rank that owns it; nothing is written locally
                from ..ops import cuda as K
                from ..parallel.symm import PushedPartial

                K.set_next_gemm_tp(comm.rs_gemm_args(plan))
                self._method.apply(self, x, bias)
                if K.take_pending_gemm_tp() is not None:
                    raise RuntimeError("linear method did not consume the pending reduce-scatter arguments")
                return PushedPartial(plan, (rows, self._n), self._compute_dtype)
        if not reduce and comm.size == 1 and comm.split_k_ok and len(x.shape) == 2 and x.shape[0] <= 256:
            # decode step on one GPU: few N tiles and a long K would leave most SMs idle, so the
            # GEMM may return its K ranges as fp32 planes that the following add + norm sums
            from ..ops import cuda as K

            K.set_next_gemm_planes(True)
            try:
                return self._method.apply(self, x, bias)
            finally:
                K.set_next_gemm_planes(False)
        y = self._method.apply(self, x, bias)
        return comm.all_reduce(y) if reduce else y
