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
_lib.bind("msgl_ar_nvls", c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_i,
                                c_ll, c_i, c_p])
_lib.bind("msgl_comm_status", c_i, [c_i])
_lib.bind("msgl_argmax_exchange", c_i, [c_p, c_ll, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_ll, c_p])

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


def agree_status(local_code: int, cpu_group, world: int) -> int:
    """MAX of the ranks' status words over the (gloo) control group."""
    if world <= 1 or cpu_group is None:
        return local_code
    t = torch.tensor([int(local_code)], dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=cpu_group)
    return int(t.item())


class MulticastBuffer:
    """One symmetric buffer that is also bound to an NVLink multicast object, set up through
    PyTorch's symmetric-memory rendezvous (``torch.distributed._symmetric_memory``): every rank gets
    its local address and one multicast address through which a ``multimem`` instruction reaches
    the same offset on all ranks (loads reduce in the switch, reductions update every copy).
    ``None`` from :meth:`create` when the platform has no multicast support."""

    def __init__(self, tensor, handle) -> None:
        self.tensor, self.handle = tensor, handle
        self.local = int(tensor.data_ptr())
        self.mc = int(handle.multicast_ptr)

    @classmethod
    def create(cls, nbytes: int, group, device) -> Optional["MulticastBuffer"]:
        try:
            import torch.distributed._symmetric_memory as symm_mem

            name = group.group_name
            enable = getattr(symm_mem, "enable_symm_mem_for_group", None)
            if enable is not None:
                try:
                    enable(name)
                except Exception:
                    pass
            t = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            hdl = symm_mem.rendezvous(t, name)
            if not int(getattr(hdl, "multicast_ptr", 0) or 0):
                return None
            t.zero_()
            torch.cuda.synchronize(device)
            hdl.barrier()
            return cls(t, hdl)
        except Exception as exc:  # no fabric / no multicast: the push form stays in use
            logger.info_rank0("NVLink multicast unavailable (%s): one-shot all-reduce stays on peer stores", exc)
            return None


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
        # vocabulary-parallel arg-max exchange: (max, index) pairs and their flags
        am_pair_bytes = 2 * world * self.max_rows * 8
        am_flag_bytes = (world * self.max_rows * 4 + 255) // 256 * 256
        self.heap = SymmetricHeap(flag_bytes + slot_bytes + am_pair_bytes + am_flag_bytes, cpu_group, rank, world)
        PtrArr = ctypes.c_void_p * world
        self._flags = PtrArr(*[p for p in self.heap.ptrs])
        self._slots = PtrArr(*[p + flag_bytes for p in self.heap.ptrs])
        self._am_pairs = PtrArr(*[p + flag_bytes + slot_bytes for p in self.heap.ptrs])
        self._am_flags = PtrArr(*[p + flag_bytes + slot_bytes + am_pair_bytes for p in self.heap.ptrs])
        self._seq = torch.zeros(self.max_rows, dtype=torch.int32, device=self.device)
        self._am_seq = torch.zeros(self.max_rows, dtype=torch.int32, device=self.device)
        self.healthy = True
        self.wait_us = ENV.COMM_WAIT_US.value
        self.oneshot_max_bytes = ENV.ONESHOT_AR_MAX_KIB.value << 10
        # in-switch reduction for the decode all-reduce when the fabric offers NVLink multicast
        self.nvls: Optional[MulticastBuffer] = None
        self._nvls_seq = None
        mode = ENV.NVLS.value
        if mode != "off" and world >= (2 if mode == "on" else 8):
            count_bytes = (self.max_rows * 4 + 255) // 256 * 256
            self.nvls = MulticastBuffer.create(count_bytes + 2 * self.max_rows * max_hidden * 2, group, self.device)
            if self.nvls is not None:
                self._nvls_seq = torch.zeros(self.max_rows, dtype=torch.int32, device=self.device)
        logger.info_rank0("peer-memory collectives ready: %d ranks, %d rows x %d, heap %.1f MiB, all-reduce by %s",
                          world, self.max_rows, max_hidden, (flag_bytes + slot_bytes) / 2 ** 20,
                          "in-switch reduction (multimem)" if self.nvls is not None else "peer stores")

    # ---- dispatch predicate ----
    def accepts(self, x: torch.Tensor) -> bool:
        return (self.healthy and x.is_cuda and x.dtype in _DT and x.dim() == 2 and x.is_contiguous()
                and x.shape[0] <= self.max_rows and x.shape[1] <= self.max_hidden and x.shape[1] % 8 == 0
                and x.numel() * 2 <= self.oneshot_max_bytes * 8)

    def _launch(self, x, residual, weight, out, out_q, out_s, eps, plus_one=False) -> None:
        from ..ops import cuda as K

        rows, hidden = x.shape
        p = lambda t: None if t is None else t.data_ptr()
        if self.nvls is not None:
            check(lib().msgl_ar_nvls(
                p(x), p(residual), p(weight), p(out), p(out_q), p(out_s), self.nvls.local, self.nvls.mc,
                self._nvls_seq.data_ptr(), self.rank, self.world, rows, hidden, self.max_rows, self.max_hidden, eps,
                int(plus_one), self.wait_us, _DT[x.dtype], torch.cuda.current_stream().cuda_stream), "ar_nvls")
            K._count("fused_allreduce", "ar_oneshot_kernel<NVLS>")
            return
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

    def vocab_argmax(self, local_logits: torch.Tensor, length: int, start: int):
        """Greedy ids from fp32 shard logits ``[rows, ld]`` (``length`` valid columns, global
        index of column 0 = ``start``): one kernel reduces the shard, exchanges (max, index)
        pairs through peer memory and picks the winner. None when the message does not fit."""
        from ..ops import cuda as K

        rows = local_logits.shape[0]
        if (not self.healthy or rows > self.max_rows or local_logits.dtype != torch.float32
                or local_logits.stride(1) != 1):
            return None
        out = torch.empty(rows, dtype=torch.int32, device=local_logits.device)
        check(lib().msgl_argmax_exchange(local_logits.data_ptr(), local_logits.stride(0), rows, int(length), int(start),
                                         out.data_ptr(), self._am_pairs, self._am_flags, self._am_seq.data_ptr(),
                                         self.rank, self.world, self.max_rows, self.wait_us,
                                         torch.cuda.current_stream().cuda_stream), "argmax_exchange")
        K._count("vocab_parallel_argmax", "argmax_exchange_kernel")
        return out

    # ---- prefill-sized messages: reduce-scatter / all-gather fused into the GEMMs ----
    def enable_row_shard(self, max_rows: int, hidden: int) -> None:
        """Collective: allocates and maps the buffers of the GEMM -> reduce-scatter -> norm ->
        all-gather -> GEMM path for up to ``max_rows`` token rows of ``hidden`` elements."""
        if getattr(self, "row_shard", None) is None and max_rows >= 128 * self.world:
            self.row_shard = RowShardFusion(self.cpu_group, self.device, self.rank, self.world, max_rows, hidden,
                                            self.wait_us)

    def rs_begin(self, rows: int, hidden: int, dtype):
        rs = getattr(self, "row_shard", None)
        if rs is None or not self.healthy or dtype not in _DT or rows <= self.max_rows or not rs.accepts(rows, hidden):
            return None
        return rs.begin(rows, dtype)

    def wait_ready(self, ready) -> None:
        from ..ops import cuda as K

        check(lib().msgl_wait_flags(ready.flags_ptr, ready.blocks,
                                    ready.seq, ready.wait_us, torch.cuda.current_stream().cuda_stream), "wait_flags")
        K._count("wait_ready", "wait_flags_kernel")

    def check_health(self) -> bool:
        """Collective over the CPU group: every rank of the group calls this on the same step.
        A bounded wait can run out on one rank only (the late peer finds its flags already
        raised), so the ranks agree on the worst status before any of them leaves the fused
        path; they then all switch to NCCL on the same step and their NCCL call sequences stay
        aligned."""
        code = agree_status(int(lib().msgl_comm_status(1)), self.cpu_group, self.world)
        if code != 0:
            self.healthy = False
            logger.warning("peer-memory collective timed out on some rank (status %d): all ranks fall back to NCCL",
                           code)
        return self.healthy

    def close(self) -> None:
        rs = getattr(self, "row_shard", None)
        if rs is not None:
            rs.close()
            self.row_shard = None
        self.nvls = None
        self.heap.close()


# ------------------------------------------------------------------------------------------
# Prefill-sized messages: GEMM -> reduce-scatter -> (add + RMSNorm) -> all-gather -> GEMM
# ------------------------------------------------------------------------------------------
_lib.bind("msgl_rs_norm_ag", c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_ll, c_i, c_i, c_i, c_i, c_i, c_i,
                                   ctypes.c_uint, ctypes.c_uint, c_f, c_i, c_i, c_ll, c_i, c_p])


_lib.bind("msgl_wait_flags", c_i, [c_p, c_i, ctypes.c_uint, c_ll, c_p])


class GemmTpArgs(ctypes.Structure):
    """Mirror of ``MsglGemmTp`` (csrc/gemm_tcgen05.cu)."""

    _fields_ = [("rs_slots", ctypes.c_void_p * 8), ("rs_flags", ctypes.c_void_p * 8), ("rs_count", ctypes.c_void_p),
                ("rs_plane", ctypes.c_longlong), ("rs_world", ctypes.c_int), ("rs_rank", ctypes.c_int),
                ("rs_flag_stride", ctypes.c_int), ("rs_ld", ctypes.c_int), ("rs_seq", ctypes.c_uint),
                ("a_ready_seq", ctypes.c_uint), ("a_ready", ctypes.c_void_p), ("wait_us", ctypes.c_longlong),
                ("order_world", ctypes.c_int)]


class ReadyRows:
    """Rows of an activation that peers are still delivering: the consumer GEMM waits for
    ``flags[block] >= seq`` per 128-row block before it stages that block."""

    __slots__ = ("flags_ptr", "seq", "world", "wait_us", "blocks")

    def __init__(self, flags_ptr: int, seq: int, world: int, wait_us: int, blocks: int) -> None:
        self.flags_ptr, self.seq, self.world, self.wait_us, self.blocks = flags_ptr, seq, world, wait_us, blocks

    def gemm_args(self) -> GemmTpArgs:
        a = GemmTpArgs()
        a.rs_world = 0
        a.a_ready = self.flags_ptr
        a.a_ready_seq = self.seq
        a.wait_us = self.wait_us
        a.order_world = self.world
        return a


class PushedPartial:
    """Stand-in for the output of a row-parallel GEMM whose epilogue pushed the partial rows to
    their owner ranks instead of writing a local tensor."""

    __slots__ = ("plan", "shape", "dtype")

    def __init__(self, plan: "RowShardPlan", shape, dtype) -> None:
        self.plan, self.shape, self.dtype = plan, shape, dtype


class RowShardPlan:
    __slots__ = ("rows", "hidden", "parity", "rs_seq", "dtype")

    def __init__(self, rows: int, hidden: int, parity: int, rs_seq: int, dtype) -> None:
        self.rows, self.hidden, self.parity, self.rs_seq, self.dtype = rows, hidden, parity, rs_seq, dtype


class RowShardFusion:
    """Symmetric buffers and sequence numbers of the prefill path. 128-row block ``b`` of the
    token rows belongs to rank ``b % world`` (its local block ``b // world``), so any row count
    that is a multiple of 128 splits evenly enough and consecutive blocks alternate owners.

    Per-rank symmetric region (``max_rows`` token rows of ``hidden`` 16-bit elements)::

        slots   2 (parity) x world (src) x blocks_per_rank x 128 x hidden 16-bit   partial rows pushed by GEMM epilogues
        rsflag  world (src) x blocks_per_rank uint32                              set by the pushing ranks
        act     2 (parity) x max_rows x hidden 16-bit (e4m3 uses the first half)  gathered normed rows
        scale   2 (parity) x max_rows fp32                                        gathered per-token scales
        ready   max_rows/128 uint32                                               set by the owning ranks
    """

    def __init__(self, cpu_group, device, rank: int, world: int, max_rows: int, hidden: int, wait_us: int) -> None:
        self.rank, self.world, self.hidden, self.wait_us = rank, world, hidden, wait_us
        self.device = torch.device(device)
        self.max_rows = (max_rows + 127) // 128 * 128
        blocks = self.max_rows // 128
        self.bpr = (blocks + world - 1) // world            # blocks per rank (upper bound)
        al = lambda n: (n + 255) // 256 * 256
        self.slot_plane = self.bpr * 128 * hidden           # elements per source plane
        self.slot_parity_bytes = world * self.slot_plane * 2
        self.off_slots = 0
        self.off_rsflag = al(2 * self.slot_parity_bytes)
        self.off_act = self.off_rsflag + al(world * self.bpr * 4)
        self.act_parity_bytes = al(self.max_rows * hidden * 2)
        self.off_scale = self.off_act + 2 * self.act_parity_bytes
        self.scale_parity_bytes = al(self.max_rows * 4)
        self.off_ready = self.off_scale + 2 * self.scale_parity_bytes
        total = self.off_ready + al(blocks * 4)
        self.heap = SymmetricHeap(total, cpu_group, rank, world)
        self.rs_count = torch.zeros(blocks + 2, dtype=torch.int32, device=self.device)
        self.blk_count = torch.zeros(self.bpr, dtype=torch.int32, device=self.device)
        self.rs_seq = 0
        self.ag_seq = 0
        self.parity = 0
        self.PtrArr = ctypes.c_void_p * world
        logger.info_rank0("row-shard fusion ready: %d ranks, %d rows x %d, heap %.1f MiB", world, self.max_rows,
                          hidden, total / 2 ** 20)

    def accepts(self, rows: int, hidden: int) -> bool:
        return hidden == self.hidden and 0 < rows <= self.max_rows and rows % 128 == 0

    # ---- producer side: arguments for the row-parallel GEMM ----
    def begin(self, rows: int, dtype) -> RowShardPlan:
        self.rs_seq = (self.rs_seq + 1) & 0xFFFFFFFF
        self.parity ^= 1
        return RowShardPlan(rows, self.hidden, self.parity, self.rs_seq, dtype)

    def gemm_args(self, plan: RowShardPlan, a_ready: Optional[ReadyRows] = None) -> GemmTpArgs:
        a = GemmTpArgs()
        for p in range(self.world):
            a.rs_slots[p] = self.heap.ptrs[p] + self.off_slots + plan.parity * self.slot_parity_bytes
            a.rs_flags[p] = self.heap.ptrs[p] + self.off_rsflag
        a.rs_count = self.rs_count.data_ptr()
        a.rs_plane = self.slot_plane
        a.rs_world, a.rs_rank, a.rs_flag_stride, a.rs_ld = self.world, self.rank, self.bpr, self.hidden
        a.rs_seq = plan.rs_seq
        a.wait_us = self.wait_us
        a.order_world = self.world
        if a_ready is not None:
            a.a_ready, a.a_ready_seq = a_ready.flags_ptr, a_ready.seq
        return a

    # ---- consumer side ----
    def finish(self, plan: RowShardPlan, residual: torch.Tensor, weight: torch.Tensor, eps: float, quant: bool,
               plus_one: bool = False):
        from ..ops import cuda as K

        rows, H = plan.rows, self.hidden
        self.ag_seq = (self.ag_seq + 1) & 0xFFFFFFFF
        par = self.ag_seq & 1
        act = [p + self.off_act + par * self.act_parity_bytes for p in self.heap.ptrs]
        scl = [p + self.off_scale + par * self.scale_parity_bytes for p in self.heap.ptrs]
        rdy = [p + self.off_ready for p in self.heap.ptrs]
        none = self.PtrArr(*([None] * self.world))
        check(lib().msgl_rs_norm_ag(
            self.heap.local + self.off_slots + plan.parity * self.slot_parity_bytes, self.heap.local + self.off_rsflag,
            residual.data_ptr(), weight.data_ptr(), none if quant else self.PtrArr(*act),
            self.PtrArr(*act) if quant else none, self.PtrArr(*scl) if quant else none, self.PtrArr(*rdy),
            self.blk_count.data_ptr(), self.slot_plane, H, self.rank, self.world, rows, self.bpr, H, plan.rs_seq,
            self.ag_seq,
            eps, int(plus_one), int(quant), self.wait_us, _DT[plan.dtype], torch.cuda.current_stream().cuda_stream),
            "rs_norm_ag")
        K._count("fused_rs_norm_ag", "rs_norm_ag_kernel")
        ready = ReadyRows(self.heap.local + self.off_ready, self.ag_seq, self.world, self.wait_us, rows // 128)
        local_act = self.heap.local + self.off_act + par * self.act_parity_bytes
        if quant:
            q = _view(local_act, (rows, H), torch.float8_e4m3fn, self.device)
            s = _view(self.heap.local + self.off_scale + par * self.scale_parity_bytes, (rows,), torch.float32,
                      self.device)
            return q, s, ready
        return _view(local_act, (rows, H), plan.dtype, self.device), None, ready

    def close(self) -> None:
        self.heap.close()


class _DevicePtr:
    """Minimal ``__cuda_array_interface__`` carrier: lets torch alias raw device memory."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _view(ptr: int, shape, dtype, device) -> torch.Tensor:
    """A tensor over raw device memory of the symmetric heap (which outlives every step)."""
    n = 1
    for d in shape:
        n *= d
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    raw = torch.as_tensor(_DevicePtr(ptr, nbytes), device=device)
    return raw.view(dtype).view(*shape)
