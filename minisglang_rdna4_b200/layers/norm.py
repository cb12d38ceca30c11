"""RMSNorm with the fused variants the decoder layer uses
(python/minisgl/layers/norm.py:61-281): plain, residual-add + norm, either of them producing
a per-token e4m3 activation for the next GEMM, and all-reduce + residual-add + norm when the
input is a tensor-parallel partial sum."""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from .. import ops
from ..parallel.comm import get_comm
from ..quant.method import ActQ
from .base import BaseOP


class RMSNorm(BaseOP):
    def __init__(self, size: int, eps: float, dtype, device, plus_one: bool = False) -> None:
        self.weight = torch.empty((size,), dtype=dtype, device=device)
        self._eps = eps
        self._plus_one = plus_one

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self._eps, self._plus_one)

    def forward_fused(self, x: torch.Tensor, residual: Optional[torch.Tensor], *, partial: bool = False,
                      quant: bool = False, to_gemm: bool = False) -> Tuple[Union[torch.Tensor, ActQ], torch.Tensor]:
        """Returns ``(normed, residual)``. ``residual`` None: the stream starts here
        (residual = x). ``partial``: ``x`` still needs the tensor-parallel all-reduce, which is
        fused with the add and the norm. ``quant``: return an ``ActQ`` pair instead of 16-bit.

        ``x`` may be a ``PushedPartial`` (the row-parallel GEMM already pushed its rows to their
        owners): this rank then reduces, adds and normalises only the rows it owns and stores
        the result into every rank's buffer. ``residual`` is from then on valid for owned rows
        only. With ``to_gemm`` the caller promises that the normed rows go straight into a
        linear layer, which waits for them block by block; otherwise the wait happens here."""
        comm = get_comm()
        if hasattr(x, "planes"):  # ops.cuda.SplitPartial: unreduced K ranges of a decode-step GEMM
            if residual is None:
                x = x.materialise()
            else:
                from ..ops import cuda as K

                out = K.rms_norm_planes(x, residual, self.weight, self._eps, self._plus_one, quant)
                return (ActQ(*out) if quant else out), residual
        if not isinstance(x, torch.Tensor):  # PushedPartial
            if residual is None:
                raise ValueError("a pushed partial sum needs a residual stream")
            q, s, ready = comm.rs_finish(x.plan, residual, self.weight, self._eps, quant, self._plus_one)
            if not to_gemm:
                comm.wait_ready(ready)
                ready = None
            if quant:
                return ActQ(q, s, ready), residual
            if ready is not None:
                q.ready = ready
            return q, residual
        if residual is None:
            if partial and comm.size > 1:
                x = comm.all_reduce(x)
            residual = x
            if quant:
                return ActQ(*ops.rms_norm_quant(x, self.weight, self._eps, None, self._plus_one)), residual
            return ops.rms_norm(x, self.weight, self._eps, self._plus_one), residual
        if partial and comm.size > 1:
            out = comm.fused_allreduce_add_rmsnorm(x, residual, self.weight, self._eps, quant)
            return (ActQ(*out) if quant else out), residual
        if quant:
            return ActQ(*ops.rms_norm_quant(x, self.weight, self._eps, residual, self._plus_one)), residual
        return ops.rms_norm_add(x, residual, self.weight, self._eps, self._plus_one), residual

    def init_dummy(self, gen=None, std: float = 0.0) -> None:
        self.weight = torch.ones_like(self.weight)
