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


class FusedEPContext(EPContext):
    """Expert-parallel exchange on the peer-memory kernels of ``csrc/ep_a2a.cu``: only the rows
    an expert owner needs are stored into its receive region (dispatch, quantised to the input
    form of the expert stack on the way out: e4m3 with one scale per token or per 128 elements),
    and only the expert outputs go back (combine, with the gate-weighted sum applied on arrival).

    Shapes are static: the regions hold ``max_tokens * top_k`` rows per source, and every step
    works under a bound ``active`` (rows any source can send this step) that is the same on all
    ranks: the agreed row count of the lock-step scheduler for eager steps, the largest graph
    bucket inside captured decode graphs. Sequence numbers and slot cursors live on the device,
    so a captured graph replays the exchange unchanged. Steps above ``max_tokens`` rows, and every
    step after a bounded wait has run out, take the gather / reduce baseline of the parent class.
    Works for DP+EP (ranks = replicas) and for EP over TP."""

    def __init__(self, group, cpu_group, rank: int, size: int, device, hidden: int, top_k: int,
                 experts_per_rank: int, max_tokens: int = 256, kind: str = "bf16") -> None:
        super().__init__(group, rank, size)
        import ctypes

        from ..env import ENV
        from ..ops._lib import bind, c_i, c_ll, c_p, lib
        from ..ops.moe_kernels import ROW_QUANT
        from .symm import SymmetricHeap

        bind("msgl_ep_region_bytes", c_ll, [c_i, c_i, c_i, c_i])
        bind("msgl_ep_dispatch", c_i, [c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p])
        bind("msgl_ep_recv_prepare", c_i, [c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_ll, c_p])
        bind("msgl_ep_gather", c_i, [c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p])
        bind("msgl_ep_return", c_i, [c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p])
        bind("msgl_ep_combine", c_i, [c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_i, c_i, c_ll, c_i, c_p])
        bind("msgl_ep_status", c_i, [c_i])
        self.device = torch.device(device)
        self.hidden, self.top_k, self.experts_per_rank = hidden, top_k, experts_per_rank
        self.kind = kind
        self.qmode = ROW_QUANT[kind] if hidden % 128 == 0 and hidden <= 8192 else 0
        self.max_tokens = max_tokens
        self.cap = max_tokens * top_k
        nbytes = int(lib().msgl_ep_region_bytes(size, self.cap, hidden, self.qmode))
        self.heap = SymmetricHeap(nbytes, cpu_group, rank, size)
        self._bases = (ctypes.c_void_p * size)(*self.heap.ptrs)
        self._state = torch.zeros(size + 4, dtype=torch.int32, device=self.device)
        self.wait_us = ENV.COMM_WAIT_US.value
        self.healthy = True
        self.fused_calls = 0
        self.static_bound: Optional[int] = None   # row bound while decode graphs are captured / replayed
        self.region_bytes = nbytes

    def step_bound(self, n_local: int) -> int:
        """Rows any rank may send in this step (identical on every rank)."""
        if self.common_tokens is not None:
            return int(self.common_tokens)
        if self.static_bound is not None:
            return int(self.static_bound)
        return self.max_tokens

    def dispatch_compute_combine(self, moe, x, topk_w, topk_ids):
        n = x.shape[0]
        bound = self.step_bound(n)
        if (not self.healthy or not x.is_cuda or bound > self.max_tokens or n > bound or n == 0 or x.dtype not in (
                torch.bfloat16, torch.float16)):
            return super().dispatch_compute_combine(moe, x, topk_w, topk_ids)
        from ..ops import cuda as K
        from ..ops import moe_kernels as MK
        from ..ops._lib import check, lib

        L = lib()
        dt = 0 if x.dtype == torch.bfloat16 else 1
        st = K._stream()
        kind, weights = moe.expert_weights()
        qmode = self.qmode
        if qmode not in (0, MK.ROW_QUANT[kind]):
            raise RuntimeError(f"expert stack of kind {kind!r} against an exchange set up for {self.kind!r}")
        active = bound * self.top_k
        x = x.contiguous()
        ids = topk_ids.contiguous()
        send_slot = torch.empty(n * self.top_k, dtype=torch.int32, device=x.device)
        check(L.msgl_ep_dispatch(self._bases, self.rank, self.size, self.cap, active, qmode, x.data_ptr(),
                                 ids.data_ptr(), send_slot.data_ptr(), self._state.data_ptr(), n, self.hidden,
                                 self.top_k, self.experts_per_rank, dt, st), "ep_dispatch")
        flat = self.size * active
        expert_ids = torch.empty(flat, dtype=torch.int32, device=x.device)
        check(L.msgl_ep_recv_prepare(self._bases, self.rank, self.size, self.cap, active, qmode, self.hidden,
                                     expert_ids.data_ptr(), self._state.data_ptr(), self.wait_us, st),
              "ep_recv_prepare")
        sorted_pair, pair_row, tile_expert, _meta = MK.moe_align(expert_ids.view(-1, 1), 0, self.experts_per_rank)
        rows = sorted_pair.numel()
        if qmode == 0:
            xq = torch.empty((rows, self.hidden), dtype=x.dtype, device=x.device)
            xsc = None
        else:
            xq = torch.empty((rows, self.hidden), dtype=torch.float8_e4m3fn, device=x.device)
            nscale = 1 if qmode == 1 else self.hidden // 128
            xsc = torch.empty((rows,) if qmode == 1 else (rows, nscale), dtype=torch.float32, device=x.device)
        check(L.msgl_ep_gather(self._bases, self.rank, self.size, self.cap, active, qmode, self.hidden,
                               sorted_pair.data_ptr(), xq.data_ptr(), None if xsc is None else xsc.data_ptr(), rows,
                               st), "ep_gather")
        if qmode == 0:
            xq, xsc = MK.quantise_rows(kind, xq)
        y = MK.run_experts_q(kind, xq, xsc, tile_expert, weights, x.dtype)
        check(L.msgl_ep_return(self._bases, self.rank, self.size, self.cap, active, qmode, self.hidden, y.data_ptr(),
                               pair_row.data_ptr(), self._state.data_ptr(), dt, st), "ep_return")
        out = torch.empty_like(x)
        check(L.msgl_ep_combine(self._bases, self.rank, self.size, self.cap, qmode, self.hidden,
                                topk_w.contiguous().data_ptr(), send_slot.data_ptr(), out.data_ptr(),
                                self._state.data_ptr(), n, self.top_k, self.wait_us, dt, st), "ep_combine")
        K._count("ep_all_to_all", "ep_dispatch+ep_recv_prepare+ep_gather+ep_return+ep_combine", 5)
        self.fused_calls += 1
        self.calls += 1
        return out

    def poll_status(self) -> int:
        """Status word of the exchange kernels on this rank (0 = no wait ran out), cleared on read.
        The lock-step loop takes the MAX over the replicas before anybody acts on it, so that all of
        them leave the fused path on the same step."""
        from ..ops._lib import lib

        return int(lib().msgl_ep_status(1)) if self.healthy else 0

    def check_health(self) -> bool:
        from ..ops._lib import lib

        code = int(lib().msgl_ep_status(1))
        if code != 0:
            self.healthy = False
        return self.healthy

    def close(self) -> None:
        self.heap.close()
