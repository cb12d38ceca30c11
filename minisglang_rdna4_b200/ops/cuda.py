"""Python wrappers of the sm_100a kernels. Every function validates shapes/dtypes, allocates
the output with PyTorch's caching allocator and launches on the current stream.

``LAUNCHES`` counts kernel launches made through this module (the benchmark reports it);
``LEDGER`` remembers which kernel served which op (printed once per op when
``MSGL_DISPATCH_LEDGER=1``, the equivalent of the reference's ``[hip-engage]`` lines,
python/minisgl/_hip_engage.py:49-71).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..env import ENV
from . import ref
from ._lib import check, lib

LAUNCHES = 0
LEDGER: Dict[str, str] = {}

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _count(op: str, kernel: str, n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n
    if op not in LEDGER:
        LEDGER[op] = kernel
        if ENV.DISPATCH_LEDGER.value:
            print(f"[sm100-engage] {op} -> {kernel}", flush=True)


# ---- guarded workspaces and the device-side bounds report (MSGL_CHECK_BOUNDS=1) ----
_GUARD_BYTES = 256
_GUARD_BYTE = 0xA5
_GUARDED: Dict[str, Tuple[torch.Tensor, int]] = {}


def workspace(name: str, numel: int, dtype, device, zero: bool = False) -> torch.Tensor:
    """A scratch buffer the kernels write. With ``MSGL_CHECK_BOUNDS=1`` it sits between two 256-byte
    guard zones filled with a byte pattern, which :func:`verify_workspaces` re-reads: a kernel that
    wrote past either end of its scratch is named instead of corrupting a neighbour silently."""
    if not ENV.CHECK_BOUNDS.value:
        return (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=device)
    item = torch.empty((), dtype=dtype).element_size()
    g = _GUARD_BYTES // item
    full = (torch.zeros if zero else torch.empty)(numel + 2 * g, dtype=dtype, device=device)
    raw = full.view(torch.uint8)
    raw[:_GUARD_BYTES] = _GUARD_BYTE
    raw[raw.numel() - _GUARD_BYTES:] = _GUARD_BYTE
    _GUARDED[f"{name}@{device}"] = (full, g)
    return full[g:g + numel]


def verify_workspaces() -> list:
    """Names of the guarded workspaces whose guard zones no longer hold the pattern (synchronises)."""
    bad = []
    for name, (full, g) in _GUARDED.items():
        raw = full.view(torch.uint8)
        lo, hi = raw[:_GUARD_BYTES], raw[raw.numel() - _GUARD_BYTES:]
        if not (bool((lo == _GUARD_BYTE).all()) and bool((hi == _GUARD_BYTE).all())):
            bad.append(name)
    return bad


def bounds_checks_enabled() -> bool:
    """True when the loaded library is the bounds-checking build."""
    from ._lib import bind, c_i

    bind("msgl_bounds_enabled", c_i, [])
    return bool(lib().msgl_bounds_enabled())


def bounds_report(max_lines: int = 64) -> list:
    """Out-of-range indices recorded by the kernels since the last call, as text lines
    ``file.cu:LINE value V limit L`` (empty with the regular library). Synchronises the device."""
    from ._lib import bind, c_i, c_p

    bind("msgl_bounds_report", c_i, [c_p, c_i, c_i])
    width = 96
    buf = ctypes.create_string_buffer(max_lines * width)
    n = int(lib().msgl_bounds_report(buf, max_lines, width))
    raw = buf.raw
    return [raw[i * width:(i + 1) * width].split(b"\0", 1)[0].decode() for i in range(min(n, max_lines))]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype} for the CUDA kernels") from None


# ------------------------------------------------------------------------------------------ elementwise
def embedding(ids, weight, vocab_start=0, vocab_len=None):
    ids = ids.to(torch.int32) if ids.dtype != torch.int32 else ids
    n = weight.shape[0] if vocab_len is None else vocab_len
    out = torch.empty((ids.numel(), weight.shape[1]), dtype=weight.dtype, device=weight.device)
    check(lib().msgl_embedding(_p(ids), _p(weight), _p(out), ids.numel(), weight.shape[1] * weight.element_size(),
                               vocab_start, n, _stream()), "embedding")
    _count("embedding", "embedding_kernel")
    return out


def _rms(x, residual, w, eps, plus_one, quant):
    assert x.is_contiguous() and x.dim() == 2
    rows, hidden = x.shape
    out = out_q = out_s = None
    if quant:
        out_q = torch.empty((rows, hidden), dtype=torch.float8_e4m3fn, device=x.device)
        out_s = torch.empty((rows,), dtype=torch.float32, device=x.device)
    else:
        out = torch.empty_like(x)
    if residual is not None:
        assert residual.is_contiguous() and residual.shape == x.shape and residual.dtype == x.dtype
    check(lib().msgl_rms_norm(_p(x), _p(residual), _p(w), _p(out), _p(out_q), _p(out_s), rows, hidden, eps,
                              int(plus_one), _dt(x), _stream()), "rms_norm")
    _count("rms_norm" + ("_add" if residual is not None else "") + ("_quant" if quant else ""), "rms_norm_kernel")
    return (out_q, out_s) if quant else out


def rms_norm_planes(part: "SplitPartial", residual, w, eps, plus_one=False, quant=False):
    """residual += (sum of the split-K planes, ascending); returns the norm of the new residual as a
    16-bit tensor or an (e4m3, scale) pair."""
    planes = part.planes
    splits, rows, hidden = planes.shape
    assert planes.is_contiguous() and residual.is_contiguous() and residual.shape == (rows, hidden)
    out = out_q = out_s = None
    if quant:
        out_q = torch.empty((rows, hidden), dtype=torch.float8_e4m3fn, device=planes.device)
        out_s = torch.empty((rows,), dtype=torch.float32, device=planes.device)
    else:
        out = torch.empty_like(residual)
    check(lib().msgl_rms_norm_planes(_p(planes), splits, _p(residual), _p(w), _p(out), _p(out_q), _p(out_s), rows,
                                     hidden, eps, int(plus_one), _dt(residual), _stream()), "rms_norm_planes")
    _count("rms_norm_add_planes" + ("_quant" if quant else ""), "rms_norm_kernel")
    return (out_q, out_s) if quant else out


def rms_norm(x, w, eps, plus_one=False):
    shape = x.shape
    return _rms(x.reshape(-1, shape[-1]), None, w, eps, plus_one, False).view(shape)


def rms_norm_add(x, residual, w, eps, plus_one=False):
    return _rms(x, residual, w, eps, plus_one, False)


def rms_norm_quant(x, w, eps, residual=None, plus_one=False):
    return _rms(x, residual, w, eps, plus_one, True)


def per_token_quant_fp8(x):
    return per_group_quant_fp8(x, 0)


def per_group_quant_fp8(x, group):
    assert x.is_contiguous() and x.dim() == 2
    rows, hidden = x.shape
    g = group or hidden
    q = torch.empty((rows, hidden), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows, hidden // g) if group else (rows,), dtype=torch.float32, device=x.device)
    check(lib().msgl_quant_fp8(_p(x), _p(q), _p(s), rows, hidden, g, _dt(x), _stream()), "quant_fp8")
    _count("quant_fp8", "quant_group_kernel")
    return q, s


_ACT = {"silu": 0, "gelu": 1, "gelu_tanh": 2}


def act_and_mul(x, kind="silu"):
    assert x.is_contiguous() and x.dim() == 2
    rows, two_i = x.shape
    out = torch.empty((rows, two_i // 2), dtype=x.dtype, device=x.device)
    check(lib().msgl_act_and_mul(_p(x), _p(out), None, None, rows, two_i // 2, _ACT[kind], _dt(x), _stream()),
          "act_and_mul")
    _count("act_and_mul", "act_mul_kernel")
    return out


def silu_and_mul_quant(x):
    assert x.is_contiguous() and x.dim() == 2
    rows, two_i = x.shape
    q = torch.empty((rows, two_i // 2), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows,), dtype=torch.float32, device=x.device)
    check(lib().msgl_act_and_mul(_p(x), None, _p(q), _p(s), rows, two_i // 2, 0, _dt(x), _stream()),
          "silu_and_mul_quant")
    _count("silu_and_mul_quant", "act_mul_quant_kernel")
    return q, s


# ------------------------------------------------------------------------------------------ rope / kv
def qk_norm_rope_store(qkv, q_w, k_w, positions, cos_sin, hq, hk, head_dim, rotary_dim, eps, k_cache, v_cache,
                       out_loc, k_scale=None, v_scale=None, interleaved=False):
    assert qkv.is_contiguous()
    t = qkv.shape[0]
    q_out = torch.empty((t, hq, head_dim), dtype=qkv.dtype, device=qkv.device)
    page_size = k_cache.shape[2]
    fp8 = k_cache.dtype == torch.float8_e4m3fn
    num_slots = k_cache.shape[0] * page_size
    check(lib().msgl_qk_norm_rope_store(
        _p(qkv), _p(q_w), _p(k_w), _p(positions), _p(cos_sin), _p(q_out), _p(k_cache), _p(v_cache), _p(out_loc),
        _p(k_scale), _p(v_scale), t, hq, hk, head_dim, rotary_dim, page_size, eps, int(interleaved), int(fp8),
        cos_sin.shape[0], num_slots, _dt(qkv), _stream()), "qk_norm_rope_store")
    _count("qk_norm_rope_store", "qk_norm_rope_store_kernel")
    return q_out


def store_kv(k, v, k_cache, v_cache, out_loc, k_scale=None, v_scale=None):
    hk, page_size, d = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    t = out_loc.numel()
    k = k.reshape(t, hk, d).contiguous()
    v = v.reshape(t, hk, d).contiguous()
    fp8 = k_cache.dtype == torch.float8_e4m3fn
    check(lib().msgl_store_kv(_p(k), _p(v), _p(k_cache), _p(v_cache), _p(out_loc), _p(k_scale), _p(v_scale), t, hk,
                              d, page_size, int(fp8), k_cache.shape[0] * page_size, _dt(k), _stream()), "store_kv")
    _count("store_kv", "store_kv_kernel")


# ------------------------------------------------------------------------------------------ attention
_KV_MAPS: Dict[Tuple, Tuple[np.ndarray, object]] = {}


def _kv_map(k_cache: torch.Tensor):
    """TMA descriptor over the pool buffer that ``k_cache`` (one layer's K plane) is a view of.
    Returns ``(descriptor bytes, layer index, number of layers)``."""
    base = k_cache._base if k_cache._base is not None else k_cache
    pages_p1, hk, ps, d = k_cache.shape
    if base.dim() == 6:
        two, layers = base.shape[0], base.shape[1]
        plane_elems = pages_p1 * hk * ps * d
        layer = (k_cache.data_ptr() - base.data_ptr()) // (plane_elems * base.element_size())
        layer = int(layer) % layers
        root = base
    else:  # a stand-alone [pages, hk, ps, d] K tensor followed by nothing: treat as one layer
        raise ValueError("paged_attention expects k_cache / v_cache to be planes of one pool buffer")
    key = (root.data_ptr(), tuple(root.shape), root.dtype)
    hit = _KV_MAPS.get(key)
    if hit is None:
        buf = np.zeros(128, dtype=np.uint8)
        check(lib().msgl_attn_make_kv_map(buf.ctypes.data, root.data_ptr(), root.element_size(), d, ps, hk,
                                          pages_p1, 2 * layers), "attn_make_kv_map")
        if len(_KV_MAPS) > 64:
            _KV_MAPS.clear()
        hit = (buf, root)
        _KV_MAPS[key] = hit
    return hit[0], layer, layers


def make_pool_buffer(num_layers, pages_plus_one, hk, page_size, d, dtype, device):
    return torch.zeros((2, num_layers, pages_plus_one, hk, page_size, d), dtype=dtype, device=device)


def attention_workspace(max_rows, hq, d, device, max_splits=16):
    return workspace("attention split partials", max_splits * max_rows * hq * (d + 1), torch.float32, device)


def choose_splits(batch, hk, max_kv, decode):
    if not decode:
        return 1
    ctas = batch * hk
    want = -(-592 // ctas)
    by_len = max(1, max_kv // 256)
    return int(max(1, min(want, by_len, 16)))


def paged_attention(q, k_cache, v_cache, block_table, cu_q, seq_lens, scale, *, causal=True, window=0, mask=None,
                    k_scale=None, v_scale=None, max_q=0, max_kv=0, decode=False, workspace=None, splits=None,
                    plan=None, tc=None, mask_window=0):
    """``plan`` (a ``PrefillPlan``) or ``tc=True`` sends a causal prefill / extend step to the
    tcgen05 kernel when it covers the shape (``tc=True`` without a plan builds the step tables from
    the device lengths, which synchronises). Without either the general kernel runs: decode and
    verification steps must not change kernels with the number of rows per request."""
    t, hq, d = q.shape
    pages_p1, hk, ps, _ = k_cache.shape
    if max_q <= 0:
        max_q = int((cu_q[1:] - cu_q[:-1]).max())
    if tc is None:
        tc = plan is not None
    if tc and prefill_attention_tc_ok(q, k_cache, causal=causal, window=window, mask=mask, decode=decode):
        if plan is None:
            plan = PrefillPlan(cu_q.cpu().numpy(), seq_lens.cpu().numpy(), q.device)
        return prefill_attention_tc(q, k_cache, v_cache, block_table, plan, scale, k_scale=k_scale, v_scale=v_scale)
    desc, layer, layers = _kv_map(k_cache)
    b = seq_lens.numel()
    if max_q <= 0:
        max_q = int((cu_q[1:] - cu_q[:-1]).max())
    if max_kv <= 0:
        max_kv = int(seq_lens.max())
    if splits is None:
        splits = choose_splits(b, hk, max_kv, decode or max_q == 1)
    if splits > 1:
        need = int(lib().msgl_attn_workspace_floats(t, hq, d, splits))
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.float32, device=q.device)
    out = torch.empty_like(q)
    fp8 = k_cache.dtype == torch.float8_e4m3fn
    mask_stride = 0
    if mask is not None:
        assert mask.dtype == torch.float32 and mask.stride(-1) == 1
        mask_stride = mask.stride(0)
        if mask_window:
            # windowed form: rows of exactly ``mask_window`` floats for the last ``mask_window`` KV
            # positions of each request (earlier positions are visible); passed as a negative stride
            assert mask.stride(0) == mask_window and mask.shape[-1] == mask_window
            mask_stride = -int(mask_window)
    check(lib().msgl_paged_attention(
        desc.ctypes.data, _p(q), _p(out), _p(block_table), block_table.stride(0), _p(cu_q), _p(seq_lens),
        _p(k_scale), _p(v_scale), _p(mask), mask_stride, _p(workspace) if splits > 1 else None,
        b, t, max_q, hq, hk, d, ps, pages_p1 - 1, layer, layers, int(fp8), int(causal), int(window), splits,
        float(scale), _dt(q), _stream()), "paged_attention")
    _count("paged_attention", "paged_attention_kernel", 2 if splits > 1 else 1)
    return out


_PLAN_RING: Dict[torch.device, list] = {}
_PLAN_RING_POS: Dict[torch.device, int] = {}


def _upload_tables(host: np.ndarray, device) -> torch.Tensor:
    """int32 tables -> device through a small ring of pinned buffers: the copy is asynchronous, so
    building the plan of the next step does not wait for the kernels of the step in flight. A
    ring slot is reused only after the event recorded behind its copy."""
    device = torch.device(device)
    if device.type != "cuda":
        return torch.from_numpy(host.copy())
    ring = _PLAN_RING.setdefault(device, [None] * 4)
    pos = _PLAN_RING_POS.get(device, 0)
    _PLAN_RING_POS[device] = pos + 1
    slot = ring[pos % 4]
    n = int(host.size)
    if slot is not None and slot[1] is not None:
        slot[1].synchronize()
    if slot is None or slot[0].numel() < n:
        slot = [torch.empty(max(n * 2, 1 << 14), dtype=torch.int32, pin_memory=True), None]
        ring[pos % 4] = slot
    slot[0].numpy()[:n] = host
    dev = torch.empty(n, dtype=torch.int32, device=device)
    dev.copy_(slot[0][:n], non_blocking=True)
    ev = torch.cuda.Event()
    ev.record()
    slot[1] = ev
    return dev


class PrefillPlan:
    """Per-step tables of the tensor-core prefill kernel: one item per (request, block of 128
    query positions), heaviest first; the request of every 128-row scratch block; per request
    the scratch offset and KV length. Built on the host from the step's lengths, one H2D copy."""

    __slots__ = ("tables", "n_items", "t_pad", "n_req", "off_blk", "off_req")

    def __init__(self, cu_q: np.ndarray, seq_lens: np.ndarray, device) -> None:
        cu_q = np.asarray(cu_q, dtype=np.int64)
        kv = np.asarray(seq_lens, dtype=np.int64)
        b = int(kv.size)
        q_len = cu_q[1:b + 1] - cu_q[:b]
        kv_pad = (kv + 127) // 128 * 128
        kv_off = np.concatenate([[0], np.cumsum(kv_pad)[:-1]]) if b else np.zeros(0, dtype=np.int64)
        self.t_pad = int(kv_pad.sum())
        self.n_req = b
        n_tiles = (q_len + 127) // 128
        req = np.repeat(np.arange(b), n_tiles)
        first = np.concatenate([[0], np.cumsum(n_tiles)[:-1]]) if b else np.zeros(0, dtype=np.int64)
        qb = np.arange(int(n_tiles.sum())) - np.repeat(first, n_tiles)
        items = np.zeros((req.size, 8), dtype=np.int32)
        rows = np.minimum(128, q_len[req] - qb * 128)
        pos0 = kv[req] - q_len[req] + qb * 128
        items[:, 0] = cu_q[req] + qb * 128
        items[:, 1] = rows
        items[:, 2] = pos0
        items[:, 3] = kv_off[req]
        items[:, 4] = (pos0 + rows + 127) // 128
        items[:, 5] = req
        items = items[np.argsort(-items[:, 4], kind="stable")]
        blk_req = np.repeat(np.arange(b), kv_pad // 128).astype(np.int32)
        req_info = np.stack([kv_off, kv], axis=1).astype(np.int32).reshape(-1)
        self.n_items = int(items.shape[0])
        self.off_blk = items.size
        self.off_req = self.off_blk + blk_req.size
        host = np.concatenate([items.reshape(-1), blk_req, req_info])
        self.tables = _upload_tables(host, device)


_TC_SCRATCH: Dict[Tuple[torch.device, torch.dtype, int], Tuple[torch.Tensor, torch.Tensor, int]] = {}


def _tc_scratch(device, dtype, hk: int, rows: int):
    """Dense K / V^T scratch shared by all layers of a step (each layer's gather overwrites it in
    stream order). Grows in steps of 8192 rows."""
    key = (device, dtype, hk)
    hit = _TC_SCRATCH.get(key)
    if hit is None or hit[2] < rows:
        cap = -(-rows // 8192) * 8192
        _TC_SCRATCH[key] = hit = (workspace(f"prefill K scratch {hk}", hk * cap * 128, dtype, device, zero=True),
                                   workspace(f"prefill V scratch {hk}", hk * cap * 128, dtype, device, zero=True), cap)
    return hit


def tc_prefill_pays(total_q: int, t_pad: int) -> bool:
    """The tensor-core path first copies every KV row the step can see into a dense 16-bit
    scratch. That is noise when the step has about as many query rows as KV rows (prefill, chunked
    prefill), but a short extend over a long cached prefix (a new chat turn over tens of thousands
    of tokens) would move several times the bytes the general kernel reads in place: such steps
    stay on the general kernel."""
    return t_pad <= 16 * max(int(total_q), 128)


def prefill_attention_tc_ok(q, k_cache, *, causal, window, mask, decode) -> bool:
    """The tcgen05 prefill kernel covers causal prefill / extend steps with head_dim 128 and an
    even number of query heads per KV head; everything else stays on the general kernel."""
    t, hq, d = q.shape
    hk = k_cache.shape[1]
    return (not decode and causal and not window and mask is None and d == 128 and hq % hk == 0
            and (hq // hk) % 2 == 0 and q.dtype in (torch.bfloat16, torch.float16) and q.stride(2) == 1
            and q.stride(1) == 128 and q.stride(0) % 8 == 0)


def prefill_attention_tc(q, k_cache, v_cache, block_table, plan: PrefillPlan, scale, *, k_scale=None, v_scale=None):
    t, hq, d = q.shape
    _, hk, ps, _ = k_cache.shape
    kc, vt, cap = _tc_scratch(q.device, q.dtype, hk, plan.t_pad)
    out = torch.empty((t, hq, d), dtype=q.dtype, device=q.device)
    tb = plan.tables
    base = tb.data_ptr()
    fp8 = k_cache.dtype == torch.float8_e4m3fn
    check(lib().msgl_attn_prefill_tc(
        _p(q), q.stride(0), _p(out), _p(k_cache), _p(v_cache), _p(kc), _p(vt), cap, plan.t_pad,
        base, plan.n_items, base + 4 * plan.off_blk, base + 4 * plan.off_req, _p(block_table), block_table.stride(0),
        _p(k_scale), _p(v_scale), t, hq, hk, ps, int(fp8), float(scale), _dt(q), _stream()), "attn_prefill_tc")
    _count("prefill_attention", "attn_prefill_tc_kernel", 2)
    return out


# ------------------------------------------------------------------------------------------ GEMM
KIND_F16, KIND_BF16, KIND_F8, KIND_MXF4 = 0, 1, 2, 3


_PENDING_TP = None
SPLIT_K = ENV.GEMM_SPLIT_K.value
_SPLITK_PLANS: Dict[Tuple[int, int, int], int] = {}
_SPLITK_COUNTERS: Dict[torch.device, torch.Tensor] = {}


def _splitk_plan(kind: int, n: int, k: int) -> int:
    key = (kind, n, k)
    s = _SPLITK_PLANS.get(key)
    if s is None:
        s = _SPLITK_PLANS[key] = int(lib().msgl_gemm_splitk_plan(kind, n, k))
    return s


def _splitk_counters(device, n: int) -> torch.Tensor:
    """Per-tile arrival counters: zero between calls (the kernel resets what it used)."""
    t = _SPLITK_COUNTERS.get(device)
    if t is None or t.numel() < n:
        t = _SPLITK_COUNTERS[device] = workspace("split-K counters", max(n, 4096), torch.int32, device, zero=True)
    return t


class SplitPartial:
    """Output of a split-K GEMM whose K ranges were not reduced: fp32 planes [splits, rows, N] that
    the next fused add + norm sums in ascending order (``rms_norm_planes``)."""

    __slots__ = ("planes", "dtype")

    def __init__(self, planes: torch.Tensor, dtype: torch.dtype) -> None:
        self.planes = planes
        self.dtype = dtype

    @property
    def shape(self):
        return self.planes.shape[1:]

    def materialise(self) -> torch.Tensor:
        out = self.planes[0].clone()
        for p in self.planes[1:]:
            out += p
        return out.to(self.dtype)


# Decode-phase row-parallel projections may hand their K ranges to the following add + norm
# unreduced. Engines that need verify rows and decode rows on one GEMM code path switch it off.
SPLIT_K_DECODE = not ENV.DISABLE_SPLIT_K_DECODE.value
_PENDING_PLANES = False


def set_next_gemm_planes(on: bool = True) -> None:
    """Ask the next GEMM call of this thread (M <= 256) to return a ``SplitPartial`` when the
    split-K plan of its (N, K) has more than one range. Consumed by exactly one call."""
    global _PENDING_PLANES
    _PENDING_PLANES = on


def set_next_gemm_tp(args) -> None:
    """Tensor-parallel fusion arguments (``parallel.symm.GemmTpArgs``) for the next GEMM call of
    this thread: push the output rows to their owner ranks and / or wait for A rows that peers
    are still delivering. Consumed by exactly one call."""
    global _PENDING_TP
    _PENDING_TP = args


def take_pending_gemm_tp():
    global _PENDING_TP
    args, _PENDING_TP = _PENDING_TP, None
    return args


def _gemm(kind, a, b, n, k, out_dtype, a_scale=None, b_scale=None, bias=None, sf_atoms=None, bn=0, max_ctas=0):
    assert a.dim() == 2 and a.stride(1) == 1 and b.is_contiguous()
    m = a.shape[0]
    tp = take_pending_gemm_tp()
    if tp is not None:
        pushes = tp.rs_world > 0
        out = None if pushes else torch.empty((m, n), dtype=out_dtype, device=a.device)
        check(lib().msgl_gemm_tp(kind, _p(a), a.stride(0), _p(b), _p(out), n, m, n, k, _p(a_scale), _p(b_scale),
                                 _p(bias), _DT[bias.dtype] if bias is not None else 0, _p(sf_atoms), _DT[out_dtype],
                                 ctypes.byref(tp), _stream()), "gemm_tp")
        _count(("gemm_f16", "gemm_bf16", "gemm_w8a8", "gemm_w4a8_mxfp4")[kind] + ("_rs" if pushes else "_ag"),
               "gemm_pair_kernel")
        return out
    global _PENDING_PLANES
    want_planes, _PENDING_PLANES = _PENDING_PLANES, False
    if want_planes and 0 < m <= 256 and bn == 0:
        splits = _splitk_plan(kind, n, k)
        if splits > 1:
            planes = torch.empty((splits, m, n), dtype=torch.float32, device=a.device)
            check(lib().msgl_gemm_splitk_planes(kind, _p(a), a.stride(0), _p(b), _p(planes), m, n, k, _p(a_scale),
                                                _p(b_scale), _p(bias), _DT[bias.dtype] if bias is not None else 0,
                                                _p(sf_atoms), splits, _stream()), "gemm_splitk_planes")
            _count(("gemm_f16", "gemm_bf16", "gemm_w8a8", "gemm_w4a8_mxfp4")[kind] + "_splitk_planes",
                   "gemm_tcgen05_kernel")
            return SplitPartial(planes, out_dtype)
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if m == 0:
        return out
    if m <= 256 and bn == 0 and SPLIT_K:
        splits = _splitk_plan(kind, n, k)
        if splits > 1:
            # small M: K ranges of one tile run on different SMs; the plan depends on (N, K) only
            mt, nt = (m + 127) // 128, (n + 127) // 128
            ws = torch.empty((splits, mt * 128, nt * 128), dtype=torch.float32, device=a.device)
            check(lib().msgl_gemm_splitk(kind, _p(a), a.stride(0), _p(b), _p(out), n, m, n, k, _p(a_scale), _p(b_scale),
                                         _p(bias), _DT[bias.dtype] if bias is not None else 0, _p(sf_atoms),
                                         _DT[out_dtype], splits, _p(ws), _p(_splitk_counters(a.device, mt * nt)),
                                         _stream()), "gemm_splitk")
            _count(("gemm_f16", "gemm_bf16", "gemm_w8a8", "gemm_w4a8_mxfp4")[kind] + "_splitk", "gemm_tcgen05_kernel")
            return out
    check(lib().msgl_gemm(kind, _p(a), a.stride(0), _p(b), _p(out), n, m, n, k, _p(a_scale), _p(b_scale), _p(bias),
                          _DT[bias.dtype] if bias is not None else 0, _p(sf_atoms), _DT[out_dtype], bn, max_ctas,
                          _stream()), "gemm")
    _count(("gemm_f16", "gemm_bf16", "gemm_w8a8", "gemm_w4a8_mxfp4")[kind], "gemm_tcgen05_kernel")
    return out


def gemm(x, w, bias=None, out_dtype=None, bn=0, max_ctas=0):
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    kind = KIND_BF16 if x2.dtype == torch.bfloat16 else KIND_F16
    if w.dtype != x2.dtype:
        raise TypeError(f"gemm: activation {x2.dtype} vs weight {w.dtype}")
    n, k = w.shape
    if n % 8:
        raise ValueError("gemm: N must be a multiple of 8")
    out = _gemm(kind, x2, w, n, k, out_dtype or x.dtype, bias=bias, bn=bn, max_ctas=max_ctas)
    if isinstance(out, SplitPartial):
        return out
    return out.view(*shape[:-1], n) if out is not None else None


def gemm_w8a8(x_q, x_scale, w_q, w_scale, out_dtype=torch.bfloat16, bias=None, bn=0):
    n, k = w_q.shape
    return _gemm(KIND_F8, x_q, w_q, n, k, out_dtype, a_scale=x_scale, b_scale=w_scale, bias=bias, bn=bn)


def gemm_w4a8_mxfp4(x_q, x_scale, w_packed, sf_atoms, out_dtype=torch.bfloat16, bias=None, bn=0):
    n, k = w_packed.shape[0], x_q.shape[-1]
    if w_packed.shape[1] * 2 != (k + 127) // 128 * 128 and w_packed.shape[1] * 2 != k:
        raise ValueError(f"gemm_w4a8_mxfp4: weights of K={w_packed.shape[1] * 2} do not match activations of K={k}")
    if w_packed.shape[1] * 2 != k and k % 128 == 0:
        raise ValueError("gemm_w4a8_mxfp4: padded weights with an unpadded K")
    if sf_atoms is None:
        raise ValueError("gemm_w4a8_mxfp4 needs the packed scale atoms (quant.mxfp4.pack_sf_atoms)")
    return _gemm(KIND_MXF4, x_q, w_packed, n, k, out_dtype, a_scale=x_scale, bias=bias, sf_atoms=sf_atoms, bn=bn)


def gemm_fp8_block(x_q, x_scale, w_q, w_scale, out_dtype=torch.bfloat16, tile_expert=None):
    """Block-scaled fp8 W8A8: ``x_q [M, K]`` e4m3 with ``x_scale [M, ceil(K/128)]`` (1 x 128 groups),
    ``w_q [N, K]`` e4m3 with ``w_scale [ceil(N/128), ceil(K/128)]`` (128 x 128 blocks). Grouped
    form: ``w_q [E, N, K]``, ``w_scale [E, N/128, ceil(K/128)]``, rows of ``x_q`` sorted by expert in
    128-row tiles and ``tile_expert [M/128]``. Every K block is accumulated on the tensor core by
    itself and promoted with its scale product (``gemm_fp8_block_kernel``)."""
    from ._lib import bind, c_i, c_ll, c_p

    if not hasattr(gemm_fp8_block, "_bound"):
        bind("msgl_gemm_fp8_block", c_i, [c_p, c_ll, c_p, c_p, c_ll, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_i, c_p])
        bind("msgl_gemm_fp8_block_status", c_i, [c_i])
        gemm_fp8_block._bound = True
    assert x_q.dtype == torch.float8_e4m3fn and w_q.dtype == torch.float8_e4m3fn
    assert x_q.dim() == 2 and x_q.stride(1) == 1 and w_q.is_contiguous()
    m, k = x_q.shape
    experts = 0
    if tile_expert is not None:
        experts, n, kw = w_q.shape
    else:
        n, kw = w_q.shape
    if kw != k:
        raise ValueError(f"gemm_fp8_block: activations of K={k} against weights of K={kw}")
    kb = (k + 127) // 128
    x_scale = x_scale.float() if x_scale.dtype != torch.float32 else x_scale
    w_scale = w_scale.float() if w_scale.dtype != torch.float32 else w_scale
    assert x_scale.is_contiguous() and x_scale.shape == (m, kb), (x_scale.shape, (m, kb))
    assert w_scale.is_contiguous() and w_scale.shape[-1] == kb and w_scale.shape[-2] == (n + 127) // 128
    out = torch.empty((m, n), dtype=out_dtype, device=x_q.device)
    check(lib().msgl_gemm_fp8_block(_p(x_q), x_q.stride(0), _p(w_q), _p(out), n, m, n, k, _p(x_scale), _p(w_scale),
                                    _p(tile_expert), experts, _DT[out_dtype], _stream()), "gemm_fp8_block")
    _count("gemm_w8a8_block" + ("_grouped" if tile_expert is not None else ""), "gemm_fp8_block_kernel")
    return out


def silu_and_mul_quant_group(x):
    """SiLU(gate) * up of ``x [rows, 2I]`` quantised to e4m3 in groups of 128 outputs:
    returns ``(q [rows, I], scales [rows, I / 128])``."""
    from ._lib import bind, c_i, c_p

    if not hasattr(silu_and_mul_quant_group, "_bound"):
        bind("msgl_silu_mul_quant_group", c_i, [c_p, c_p, c_p, c_i, c_i, c_i, c_p])
        silu_and_mul_quant_group._bound = True
    assert x.is_contiguous() and x.dim() == 2
    rows, two_i = x.shape
    inter = two_i // 2
    q = torch.empty((rows, inter), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((rows, inter // 128), dtype=torch.float32, device=x.device)
    check(lib().msgl_silu_mul_quant_group(_p(x), _p(q), _p(s), rows, inter, _dt(x), _stream()), "silu_mul_quant_group")
    _count("silu_and_mul_quant_group", "silu_mul_quant_group_kernel")
    return q, s


W4_EXPAND_ROWS = 256
_W4_SCRATCH: Dict[Tuple[torch.device, torch.dtype], torch.Tensor] = {}


def _w4_scratch(device, dtype, elems: int) -> torch.Tensor:
    key = (device, dtype)
    t = _W4_SCRATCH.get(key)
    if t is None or t.numel() < elems:
        t = _W4_SCRATCH[key] = workspace("4-bit expansion scratch", elems, dtype, device)
    return t


def gemm_w4a16(x, w_packed, scales_t, zeros_t=None, channel=None, group=128, nvfp4=False, bias=None, out_dtype=None):
    """``x @ dequant(W).T`` with W kept 4-bit in HBM (``gemm_w4a16_kernel``): ``w_packed [N, K/2]`` bytes
    (low nibble = even k), ``scales_t [K/group, N]`` fp32 with ``zeros_t`` of the same shape (integer
    formats: ``w = (code - zero) * scale``), or e4m3 bytes with a per-channel fp32 factor ``channel [N]``
    (NVFP4: ``w = e2m1(code) * scale * channel``). Activations stay 16-bit."""
    from ._lib import bind, c_i, c_ll, c_p

    if not hasattr(gemm_w4a16, "_bound"):
        bind("msgl_gemm_w4a16", c_i, [c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_p, c_ll, c_i, c_i, c_i, c_i, c_i, c_i, c_i,
                                      c_p])
        bind("msgl_gemm_w4a16_status", c_i, [c_i])
        bind("msgl_w4_expand", c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p])
        gemm_w4a16._bound = True
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    m, k = x2.shape
    n = w_packed.shape[0]
    assert w_packed.dtype == torch.uint8 and w_packed.is_contiguous() and w_packed.shape[1] * 2 == k
    assert scales_t.is_contiguous() and scales_t.shape == (k // group, n)
    out_dtype = out_dtype or x.dtype
    if m > W4_EXPAND_ROWS:
        # many rows (prefill): expand the matrix once into a scratch shared by all layers, then the
        # ordinary GEMM; the in-kernel expansion would repeat per 128-row tile
        scratch = _w4_scratch(x.device, x.dtype, n * k)
        check(lib().msgl_w4_expand(_p(w_packed), _p(scales_t), _p(zeros_t), _p(channel), _p(scratch), n, k, group,
                                   int(nvfp4), _dt(x2), _stream()), "w4_expand")
        _count("w4_expand", "w4_expand_kernel")
        # the scratch is written by the kernel just ahead: no weight fetch before the dependency wait
        prev = gemm_static_weights(False)
        try:
            out = _gemm(KIND_BF16 if x.dtype == torch.bfloat16 else KIND_F16, x2, scratch[: n * k].view(n, k), n, k,
                        out_dtype, bias=bias)
        finally:
            gemm_static_weights(prev)
        return out.view(*shape[:-1], n) if out is not None else None
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(lib().msgl_gemm_w4a16(_p(x2), x2.stride(0), _p(w_packed), _p(scales_t), _p(zeros_t), _p(channel), _p(bias),
                                _p(out), n, m, n, k, group, int(nvfp4), _dt(x2), _DT[out_dtype], _stream()),
          "gemm_w4a16")
    _count("gemm_w4a16_nvfp4" if nvfp4 else "gemm_w4a16_int4", "gemm_w4a16_kernel")
    return out.view(*shape[:-1], n)


def gemm_w4a16_status(reset=True) -> int:
    from ._lib import bind, c_i

    bind("msgl_gemm_w4a16_status", c_i, [c_i])
    return int(lib().msgl_gemm_w4a16_status(int(reset)))


def gemm_status(reset=True) -> int:
    return int(lib().msgl_gemm_status(int(reset)))


def gemm_pair_mode(mode: int) -> int:
    """Tile policy of the GEMM family: 0 = CTA-pair kernel (256 x 256 tiles, two SMs per tile)
    above 256 rows, 1 = single-CTA kernel always, 2 = CTA-pair kernel always. Returns the
    previous setting."""
    return int(lib().msgl_gemm_pair_mode(int(mode)))


def gemm_static_weights(on) -> int:
    """Promise that the weight operands of all GEMM calls from now on are model parameters
    (written long before the kernels in flight): the decode GEMMs then fetch their first weight
    tiles while the kernel ahead of them is still running (1), and also request the rest of their
    first work item's weight stream into L2 (2). Returns the previous setting."""
    return int(lib().msgl_gemm_static_weights(int(on)))


def set_pdl(on: bool) -> int:
    """Programmatic dependent launch of the library's kernels (on by default; ``MSGL_PDL=0``
    switches it off). Returns the previous setting."""
    return int(lib().msgl_set_pdl(int(on)))


def decode_attention_stages(stages: int) -> None:
    """Depth of the fp8 decode kernel's TMA ring (2-4 stages of 64 tokens)."""
    lib().msgl_attn_decode_stages(int(stages))


def force_general_decode_attention(on: bool) -> None:
    """Route single-query batches through the general attention kernel. Speculative decoding
    sets this: verification rows run on the general kernel, and greedy output is only
    bit-identical to plain decoding when the decode rows take the same code path."""
    lib().msgl_attn_force_general_decode(int(on))


def gemm_fp8_block_status(reset=True) -> int:
    from ._lib import bind, c_i

    bind("msgl_gemm_fp8_block_status", c_i, [c_i])
    return int(lib().msgl_gemm_fp8_block_status(int(reset)))


def attn_status(reset=True) -> int:
    a = int(lib().msgl_attn_status(int(reset)))
    b = int(lib().msgl_attn_tc_status(int(reset)))
    return a or b


# ------------------------------------------------------------------------------------------ sampling
def argmax(logits):
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1
    rows, vocab = logits.shape
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(lib().msgl_argmax(_p(logits), _p(out), rows, vocab, logits.stride(0), _stream()), "argmax")
    _count("argmax", "argmax_kernel")
    return out


def sample(logits, temperatures, top_k=None, top_p=None, min_p=None, generator=None, uniform=None):
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1
    rows, vocab = logits.shape
    if uniform is None:
        uniform = torch.rand((rows,), dtype=torch.float32, device=logits.device, generator=generator)
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(lib().msgl_sample(_p(logits), logits.stride(0), _p(temperatures), _p(top_k), _p(top_p), _p(min_p),
                            _p(uniform), _p(out), rows, vocab, _stream()), "sample")
    _count("sample", "sample_kernel")
    return out


# ------------------------------------------------------------------------------------------ MoE (composed)
def moe_route(router_logits, top_k, renormalize, scoring="softmax", bias=None, scale=1.0, counts=None, e_start=0,
              e_local=None):
    from . import moe_kernels

    return moe_kernels.moe_route(router_logits, top_k, renormalize, scoring, scale, counts, e_start, e_local, bias)


def moe_forward(x, w13, w2, topk_w, topk_ids, expert_offset=0, counts=None):
    from . import moe_kernels

    return moe_kernels.moe_forward(x, w13, w2, topk_w, topk_ids, expert_offset, counts)


# ------------------------------------------------------------------------------------------ gated delta net
def _bind_gdn():
    from ._lib import bind, c_f, c_i, c_ll, c_p

    if getattr(_bind_gdn, "done", False):
        return
    bind("msgl_gdn_conv1d", c_i, [c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p, c_i, c_p])
    bind("msgl_mamba2_scan", c_i, [c_p, c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_f,
                                   c_i, c_p])
    bind("msgl_rms_norm_gate_first", c_i, [c_p, c_p, c_ll, c_p, c_p, c_i, c_i, c_i, c_f, c_i, c_p])
    bind("msgl_relu2", c_i, [c_p, c_p, c_ll, c_i, c_p])
    bind("msgl_gdn_recurrent", c_i, [c_p, c_p, c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i,
                                     c_p])
    bind("msgl_rms_norm_gated", c_i, [c_p, c_p, c_ll, c_i, c_p, c_p, c_i, c_i, c_f, c_i, c_p])
    _bind_gdn.done = True


def gdn_conv1d(x, weight, conv_state, cu_q, slots, has_state, bias=None):
    """Depthwise causal conv (4 taps, optional bias) + SiLU over packed sequences; ``x [T, C]`` may be a
    column slice of a wider projection (row stride = its leading dimension). Updates ``conv_state``."""
    _bind_gdn()
    assert x.dim() == 2 and x.stride(1) == 1 and weight.is_contiguous() and conv_state.is_contiguous()
    t, c = x.shape
    out = torch.empty((t, c), dtype=x.dtype, device=x.device)
    check(lib().msgl_gdn_conv1d(_p(x), x.stride(0), _p(weight), _p(conv_state), _p(cu_q), _p(slots), _p(has_state),
                                _p(out), cu_q.numel() - 1, c, weight.shape[1], _p(bias), _dt(x), _stream()), "gdn_conv1d")
    _count("gdn_conv1d", "gdn_conv1d_kernel")
    return out


def gdn_recurrent(qkv, a, b, a_log, dt_bias, state, cu_q, slots, has_state, hk, hv, dk, dv):
    """Gated delta rule over packed sequences. ``qkv [T, 2*hk*dk + hv*dv]`` (after the convolution),
    ``a, b [T, hv]`` raw gate projections (column slices allowed, same row stride), ``state
    [slots, hv, dk, dv]`` fp32 updated in place. Returns ``[T, hv, dv]``."""
    _bind_gdn()
    assert qkv.is_contiguous() and a.stride(1) == 1 and b.stride(1) == 1 and a.stride(0) == b.stride(0)
    assert state.dtype == torch.float32 and state.is_contiguous()
    t = qkv.shape[0]
    out = torch.empty((t, hv, dv), dtype=qkv.dtype, device=qkv.device)
    check(lib().msgl_gdn_recurrent(_p(qkv), _p(a), _p(b), a.stride(0), _p(a_log), _p(dt_bias), _p(state), _p(cu_q),
                                   _p(slots), _p(has_state), _p(out), cu_q.numel() - 1, hk, hv, dk, dv, _dt(qkv),
                                   _stream()), "gdn_recurrent")
    _count("gdn_recurrent", "gdn_recurrent_kernel")
    return out


def mamba2_scan(xbc, dt, a_log, d_skip, dt_bias, state, cu_q, slots, has_state, heads, groups, head_dim, state_size,
                dt_min=0.0):
    """Selective state-space recurrence over packed sequences. ``xbc [T, H*P + 2*G*N]`` (after the
    convolution: x heads, B groups, C groups), ``dt [T, H]`` raw step sizes (a column slice is fine),
    ``state [slots, H, P, N]`` fp32 updated in place. Returns ``[T, H, P]``."""
    _bind_gdn()
    assert xbc.is_contiguous() and dt.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
    t = xbc.shape[0]
    out = torch.empty((t, heads, head_dim), dtype=xbc.dtype, device=xbc.device)
    check(lib().msgl_mamba2_scan(_p(xbc), _p(dt), dt.stride(0), _p(a_log), _p(d_skip), _p(dt_bias), _p(state), _p(cu_q),
                                 _p(slots), _p(has_state), _p(out), cu_q.numel() - 1, heads, groups, head_dim,
                                 state_size, float(dt_min), _dt(xbc), _stream()), "mamba2_scan")
    _count("mamba2_scan", "mamba2_scan_kernel")
    return out


def rms_norm_gate_first(x, z, w, eps, group):
    """``w * norm_group(x * silu(z))``: ``x [T, D]`` contiguous, ``z [T, D]`` (a column slice is fine)."""
    _bind_gdn()
    t, d = x.shape
    assert x.is_contiguous() and z.stride(1) == 1
    out = torch.empty_like(x)
    check(lib().msgl_rms_norm_gate_first(_p(x), _p(z), z.stride(0), _p(w), _p(out), t, d, group, eps, _dt(x), _stream()),
          "rms_norm_gate_first")
    _count("rms_norm_gate_first", "rms_norm_gate_first_kernel")
    return out


def relu2(x):
    _bind_gdn()
    x = x.contiguous()
    out = torch.empty_like(x)
    check(lib().msgl_relu2(_p(x), _p(out), x.numel(), _dt(x), _stream()), "relu2")
    _count("relu2", "relu2_kernel")
    return out


def rms_norm_gated(x, z, w, eps):
    """``norm(x) * w * silu(z)`` per head: ``x [T, heads, D]`` contiguous, ``z [T, heads * D]`` (a column
    slice of a wider projection is fine)."""
    _bind_gdn()
    t, heads, d = x.shape
    assert x.is_contiguous() and z.stride(1) == 1
    out = torch.empty_like(x)
    check(lib().msgl_rms_norm_gated(_p(x), _p(z), z.stride(0), heads, _p(w), _p(out), t * heads, d, eps, _dt(x),
                                    _stream()), "rms_norm_gated")
    _count("rms_norm_gated", "rms_norm_gated_kernel")
    return out
