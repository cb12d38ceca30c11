"""Symmetric peer-memory runtime and the fused collectives built on it.

At boot every rank allocates one device buffer (data slots + flag words), exports it with a
CUDA IPC handle, gathers all handles over the gloo control group and maps its peers' buffers.
The kernels in ``csrc/comm.cu`` then address peer memory directly over NVLink. The reference
does the same for two PCIe peers (python/minisgl/distributed/impl.py:290-320,455-520); here the
world is up to eight NVSwitch-connected GPUs.

Layout of one rank's buffer::

    [ flags   : nranks * max_rows uint32 ]                      raised by peers, per (src, row)
    [ slots   : 2 (parity) * nranks (src) * max_rows * max_hidden 16-bit ]

Health: every device-side wait is bounded. ``check_health`` reads the status word; a non-zero
value marks the fast path unhealthy and the communicator falls back to NCCL for the rest of
the process (python/minisgl/distributed/impl.py:317-320 falls back silently at set-up only).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..env import ENV
from ..ops import _lib
from ..ops._lib import c_f, c_i, c_ll, c_p, check, lib
from ..utils import init_logger

logger = init_logger(__name__)

_lib.bind("msgl_symm_alloc", c_p, [c_ll])
_lib.bind("msgl_symm_free", c_i, [c_p])
_lib.bind("msgl_ipc_get_handle", c_i, [c_p, c_p])
_lib.bind("msgl_ipc_open", c_p, [c_p])
_lib.bind("msgl_ipc_close", c_i, [c_p])
_lib.bind("msgl_ar_oneshot", c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i,
                                   c_f, c_i, c_ll, c_i, c_p])
_lib.bind("msgl_comm_status", c_i, [c_i])

_DT = {torch.bfloat16: 0, torch.float16: 1}


class SymmetricHeap:
    """One IPC-shared device buffer per rank, mapped on every rank."""

    def __init__(self, nbytes: int, cpu_group: dist.ProcessGroup, rank: int, world: int) -> None:
        L = lib()
        self.rank, self.world, self.nbytes = rank, world, nbytes
        self.local = L.msgl_symm_alloc(nbytes)
        if not self.local:
            raise RuntimeError("symmetric heap allocation failed: " + L.msgl_last_error().decode())
        handle = (ctypes.c_ubyte * 64)()
        check(L.msgl_ipc_get_handle(self.local, handle), "ipc_get_handle")
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=cpu_group)
        self.ptrs: List[int] = []
        for r, h in enumerate(handles):
            if r == rank:
                self.ptrs.append(self.local)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            p = L.msgl_ipc_open(buf)
            if not p:
                raise RuntimeError(f"cannot map rank {r}'s buffer: " + L.msgl_last_error().decode())
            self.ptrs.append(p)
        dist.barrier(group=cpu_group)

    def close(self) -> None:
        L = lib()
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                L.msgl_ipc_close(p)
        if self.local:
            L.msgl_symm_free(self.local)
        self.ptrs, self.local = [], None


class SymmetricCollectives:
    name = "symm"

    def __init__(self, group: dist.ProcessGroup, cpu_group: dist.ProcessGroup, device, rank: int, world: int,
                 max_rows: int = 512, max_hidden: int = 8192) -> None:
        if world > 8:
            raise ValueError("the peer-memory collectives support up to 8 ranks")
        self.group, self.cpu_group = group, cpu_group
        self.rank, self.world = rank, world
        self.device = torch.device(device)
        self.max_rows, self.max_hidden = max_rows, max_hidden
        budget = ENV.SYMM_HEAP_MIB.value << 20
        flag_bytes = world * max_rows * 4
        flag_bytes = (flag_bytes + 255) // 256 * 256
        slot_bytes = 2 * world * max_rows * max_hidden * 2
        while flag_bytes + slot_bytes > budget and self.max_rows > 16:
            self.max_rows //= 2
            flag_bytes = (world * self.max_rows * 4 + 255) // 256 * 256
            slot_bytes = 2 * world * self.max_rows * max_hidden * 2
        self.heap = SymmetricHeap(flag_bytes + slot_bytes, cpu_group, rank, world)
        PtrArr = ctypes.c_void_p * world
        self._flags = PtrArr(*[p for p in self.heap.ptrs])
        self._slots = PtrArr(*[p + flag_bytes for p in self.heap.ptrs])
        self._seq = torch.zeros(self.max_rows, dtype=torch.int32, device=self.device)
        self.healthy = True
        self.wait_us = ENV.COMM_WAIT_US.value
        self.oneshot_max_bytes = ENV.ONESHOT_AR_MAX_KIB.value << 10
        logger.info_rank0("peer-memory collectives ready: %d ranks, %d rows x %d, heap %.1f MiB",
                          world, self.max_rows, max_hidden, (flag_bytes + slot_bytes) / 2 ** 20)

    # ---- dispatch predicate ----
    def accepts(self, x: torch.Tensor) -> bool:
        return (self.healthy and x.is_cuda and x.dtype in _DT and x.dim() == 2 and x.is_contiguous()
                and x.shape[0] <= self.max_rows and x.shape[1] <= self.max_hidden and x.shape[1] % 8 == 0
                and x.numel() * 2 <= self.oneshot_max_bytes * 8)

    def _launch(self, x, residual, weight, out, out_q, out_s, eps, plus_one=False) -> None:
        from ..ops import cuda as K

        rows, hidden = x.shape
        p = lambda t: None if t is None else t.data_ptr()
        check(lib().msgl_ar_oneshot(
            p(x), p(residual), p(weight), p(out), p(out_q), p(out_s), self._slots, self._flags, self._seq.data_ptr(),
            self.rank, self.world, rows, hidden, self.max_rows, self.max_hidden, eps, int(plus_one), self.wait_us,
            _DT[x.dtype], torch.cuda.current_stream().cuda_stream), "ar_oneshot")
        K._count("fused_allreduce", "ar_oneshot_kernel")

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        self._launch(x, None, None, x, None, None, 0.0)
        return x

    def fused_allreduce_add_rmsnorm(self, x, residual, weight, eps, quant=False):
        rows, hidden = x.shape
        if quant:
            q = torch.empty((rows, hidden), dtype=torch.float8_e4m3fn, device=x.device)
            s = torch.empty((rows,), dtype=torch.float32, device=x.device)
            self._launch(x, residual, weight, None, q, s, eps)
            return q, s
        out = torch.empty_like(x)
        self._launch(x, residual, weight, out, None, None, eps)
        return out

    def check_health(self) -> bool:
        code = int(lib().msgl_comm_status(1))
        if code != 0:
            self.healthy = False
            logger.warning("peer-memory collective timed out (status %d): falling back to NCCL", code)
        return self.healthy

    def close(self) -> None:
        self.heap.close()
