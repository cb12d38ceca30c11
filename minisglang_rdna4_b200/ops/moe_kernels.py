"""Python side of the fused MoE path: routing kernel, alignment to 128-row tiles, permute,
two grouped tcgen05 GEMMs with SiLU·mul between them, weighted combine."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import _lib
from . import cuda as K
from ._lib import c_f, c_i, c_ll, c_p, check, lib

_lib.bind("msgl_moe_route", c_i, [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_f, c_i, c_i, c_i, c_p])
_lib.bind("msgl_moe_align", c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_p])
_lib.bind("msgl_moe_permute", c_i, [c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p])
_lib.bind("msgl_moe_combine", c_i, [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p])
_lib.bind("msgl_gemm_grouped", c_i, [c_i, c_p, c_ll, c_p, c_p, c_ll, c_i, c_i, c_i, c_p, c_i, c_p, c_p, c_i, c_i, c_p])

BLOCK = 128
_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def moe_route(router_logits, top_k, renormalize, scoring="softmax", scale=1.0, counts=None, e_start=0, e_local=None,
              bias=None):
    """Softmax / sigmoid scores, top-k by score (+ selection ``bias`` when given), optional
    renormalisation, in one launch. ``counts [e_local]`` (int32), when given, receives the number
    of tokens routed to every local expert, which is what the alignment step needs."""
    t, e = router_logits.shape
    assert router_logits.is_contiguous()
    w = torch.empty((t, top_k), dtype=torch.float32, device=router_logits.device)
    ids = torch.empty((t, top_k), dtype=torch.int32, device=router_logits.device)
    if bias is not None:
        bias = bias.float().contiguous()
    check(lib().msgl_moe_route(router_logits.data_ptr(), None if bias is None else bias.data_ptr(), w.data_ptr(),
                               ids.data_ptr(), None if counts is None else counts.data_ptr(), t, e, top_k,
                               int(renormalize),
                               int(scoring != "softmax"), float(scale), e_start, e if e_local is None else e_local,
                               _DT[router_logits.dtype], K._stream()), "moe_route")
    K._count("moe_route", "moe_route_kernel")
    return w, ids


def max_sorted_rows(tokens: int, top_k: int, e_local: int) -> int:
    rows = tokens * top_k + e_local * (BLOCK - 1)
    return (rows + BLOCK - 1) // BLOCK * BLOCK


def moe_align(topk_ids, e_start: int, e_local: int, counts=None):
    """Returns ``(sorted_pair [R], pair_row [T*k], tile_expert [R/128], meta [2])`` with R the
    worst-case padded row count (static for a given T, k, E). ``counts`` = tokens per local expert
    when the routing kernel already produced them."""
    t, k = topk_ids.shape
    dev = topk_ids.device
    rows = max_sorted_rows(t, k, e_local)
    if counts is None:
        counts = torch.zeros(e_local, dtype=torch.int32, device=dev)
        flat = topk_ids.reshape(-1).long() - e_start
        ok = (flat >= 0) & (flat < e_local)
        counts.index_add_(0, flat.clamp(0, e_local - 1), ok.to(torch.int32))
    return _align_with_counts(topk_ids, counts, e_start, e_local, rows)


def _align_with_counts(topk_ids, counts, e_start, e_local, rows):
    t, k = topk_ids.shape
    dev = topk_ids.device
    offsets = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
    cursor = torch.empty(e_local, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(rows // BLOCK, dtype=torch.int32, device=dev)
    meta = torch.empty(2, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(rows, dtype=torch.int32, device=dev)
    pair_row = torch.empty(t * k, dtype=torch.int32, device=dev)
    check(lib().msgl_moe_align(topk_ids.data_ptr(), counts.data_ptr(), offsets.data_ptr(), cursor.data_ptr(),
                               tile_expert.data_ptr(), meta.data_ptr(), sorted_pair.data_ptr(), pair_row.data_ptr(),
                               t, k, e_start, e_local, rows, BLOCK, K._stream()), "moe_align")
    K._count("moe_align", "moe_offsets_kernel+moe_scatter_kernel", 2)
    return sorted_pair, pair_row, tile_expert, meta


def gemm_grouped(a, b, tile_expert, out_dtype=None, bn=0):
    """``a [R, K]`` (expert-sorted rows, R % 128 == 0), ``b [E, N, K]`` → ``[R, N]``."""
    e, n, k = b.shape
    r = a.shape[0]
    out = torch.empty((r, n), dtype=out_dtype or a.dtype, device=a.device)
    kind = K.KIND_BF16 if a.dtype == torch.bfloat16 else K.KIND_F16
    check(lib().msgl_gemm_grouped(kind, a.data_ptr(), a.stride(0), b.data_ptr(), out.data_ptr(), n, r, n, k,
                                  tile_expert.data_ptr(), e, None, None, _DT[out.dtype], bn, K._stream()),
          "gemm_grouped")
    K._count("moe_gemm_grouped", "gemm_tcgen05_kernel")
    return out


def moe_forward(x, w13, w2, topk_w, topk_ids, expert_offset=0, counts=None):
    t, h = x.shape
    e_local = w13.shape[0]
    k = topk_ids.shape[1]
    sorted_pair, pair_row, tile_expert, _meta = moe_align(topk_ids, expert_offset, e_local, counts)
    rows = sorted_pair.numel()
    xs = torch.empty((rows, h), dtype=x.dtype, device=x.device)
    check(lib().msgl_moe_permute(x.data_ptr(), sorted_pair.data_ptr(), xs.data_ptr(), h, k, rows, _DT[x.dtype],
                                 K._stream()), "moe_permute")
    K._count("moe_permute", "moe_permute_kernel")
    hcur = gemm_grouped(xs, w13, tile_expert)
    act = K.act_and_mul(hcur)
    y = gemm_grouped(act, w2, tile_expert)
    out = torch.empty_like(x)
    check(lib().msgl_moe_combine(y.data_ptr(), topk_w.data_ptr(), pair_row.data_ptr(), out.data_ptr(), t, h, k,
                                 _DT[x.dtype], K._stream()), "moe_combine")
    K._count("moe_combine", "moe_combine_kernel")
    return out


def moe_forward_plain(x, w1, w2, topk_w, topk_ids, expert_offset=0, counts=None, act="relu2"):
    """Non-gated experts (``down(act(up x))``, Nemotron-H): ``w1 [E, I, H]``, ``w2 [E, H, I]``, 16-bit."""
    if act != "relu2":
        raise ValueError(f"non-gated experts with activation {act!r}")
    t, h = x.shape
    k = topk_ids.shape[1]
    sorted_pair, pair_row, tile_expert, _meta = moe_align(topk_ids, expert_offset, w1.shape[0], counts)
    xs = _permute(x, sorted_pair, k)
    y = gemm_grouped(K.relu2(gemm_grouped(xs, w1, tile_expert)), w2, tile_expert)
    return _combine(y, topk_w, pair_row, x, k)


def gemm_grouped_w4a8(a_q, a_scale, b_packed, sf_atoms, tile_expert, out_dtype=torch.bfloat16, bn=0):
    """MXFP4 experts: ``a_q [R, K]`` e4m3 rows (expert-sorted, R % 128 == 0) with per-row scales,
    ``b_packed [E, N, K/2]`` e2m1 pairs, ``sf_atoms [E, ceil(N/128), ceil(K/128), 32, 4, 4]`` → ``[R, N]``."""
    e, n, k2 = b_packed.shape
    r = a_q.shape[0]
    out = torch.empty((r, n), dtype=out_dtype, device=a_q.device)
    check(lib().msgl_gemm_grouped(K.KIND_MXF4, a_q.data_ptr(), a_q.stride(0), b_packed.data_ptr(), out.data_ptr(), n,
                                  r, n, k2 * 2, tile_expert.data_ptr(), e, a_scale.data_ptr(), sf_atoms.data_ptr(),
                                  _DT[out_dtype], bn, K._stream()), "gemm_grouped_w4a8")
    K._count("moe_gemm_grouped_w4a8", "gemm_tcgen05_kernel")
    return out


def moe_forward_w4a8(x, w13_packed, w13_atoms, w2_packed, w2_atoms, topk_w, topk_ids, expert_offset=0):
    """Expert MLPs with 4-bit weights and e4m3 activations: permute → per-row quantise →
    grouped block-scaled GEMM → SiLU·mul fused with the next quantiser → grouped GEMM → combine."""
    t, h = x.shape
    e_local = w13_packed.shape[0]
    k = topk_ids.shape[1]
    sorted_pair, pair_row, tile_expert, _meta = moe_align(topk_ids, expert_offset, e_local)
    rows = sorted_pair.numel()
    xs = torch.empty((rows, h), dtype=x.dtype, device=x.device)
    check(lib().msgl_moe_permute(x.data_ptr(), sorted_pair.data_ptr(), xs.data_ptr(), h, k, rows, _DT[x.dtype],
                                 K._stream()), "moe_permute")
    K._count("moe_permute", "moe_permute_kernel")
    xq, xsc = K.per_token_quant_fp8(xs)
    hcur = gemm_grouped_w4a8(xq, xsc, w13_packed, w13_atoms, tile_expert, x.dtype)
    aq, asc = K.silu_and_mul_quant(hcur)
    y = gemm_grouped_w4a8(aq, asc, w2_packed, w2_atoms, tile_expert, x.dtype)
    out = torch.empty_like(x)
    check(lib().msgl_moe_combine(y.data_ptr(), topk_w.data_ptr(), pair_row.data_ptr(), out.data_ptr(), t, h, k,
                                 _DT[x.dtype], K._stream()), "moe_combine")
    K._count("moe_combine", "moe_combine_kernel")
    return out


_lib.bind("msgl_gemm_grouped_w8a8", c_i, [c_p, c_ll, c_p, c_p, c_ll, c_i, c_i, c_i, c_p, c_i, c_p, c_p, c_i, c_i, c_p])


def _permute(x, sorted_pair, k):
    rows, h = sorted_pair.numel(), x.shape[1]
    xs = torch.empty((rows, h), dtype=x.dtype, device=x.device)
    check(lib().msgl_moe_permute(x.data_ptr(), sorted_pair.data_ptr(), xs.data_ptr(), h, k, rows, _DT[x.dtype],
                                 K._stream()), "moe_permute")
    K._count("moe_permute", "moe_permute_kernel")
    return xs


def _combine(y, topk_w, pair_row, like, k):
    t, h = like.shape
    out = torch.empty_like(like)
    check(lib().msgl_moe_combine(y.data_ptr(), topk_w.data_ptr(), pair_row.data_ptr(), out.data_ptr(), t, h, k,
                                 _DT[like.dtype], K._stream()), "moe_combine")
    K._count("moe_combine", "moe_combine_kernel")
    return out


def gemm_grouped_w8a8(a_q, a_scale, b_q, b_scale, tile_expert, out_dtype=torch.bfloat16, bn=0):
    """fp8 experts with per-channel scales: ``a_q [R, K]`` e4m3 rows (expert-sorted) with per-row
    scales, ``b_q [E, N, K]`` e4m3, ``b_scale [E, N]`` fp32 → ``[R, N]``."""
    e, n, k = b_q.shape
    r = a_q.shape[0]
    out = torch.empty((r, n), dtype=out_dtype, device=a_q.device)
    check(lib().msgl_gemm_grouped_w8a8(a_q.data_ptr(), a_q.stride(0), b_q.data_ptr(), out.data_ptr(), n, r, n, k,
                                       tile_expert.data_ptr(), e, a_scale.data_ptr(), b_scale.data_ptr(),
                                       _DT[out_dtype], bn, K._stream()), "gemm_grouped_w8a8")
    K._count("moe_gemm_grouped_w8a8", "gemm_tcgen05_kernel")
    return out


# How the rows entering the expert MLPs are quantised, per kind of expert stack:
# 0 = 16-bit rows, 1 = e4m3 + one scale per token, 2 = e4m3 + one scale per 128 elements
ROW_QUANT = {"bf16": 0, "mxfp4": 1, "fp8_channel": 1, "fp8_block": 2}


def quantise_rows(kind: str, xs):
    mode = ROW_QUANT[kind]
    if mode == 0:
        return xs, None
    if mode == 1:
        return K.per_token_quant_fp8(xs)
    return K.per_group_quant_fp8(xs, 128)


def run_experts_q(kind: str, xq, xsc, tile_expert, weights, out_dtype):
    """The two expert GEMMs with SiLU·mul (+ re-quantisation) between them, on expert-sorted rows
    that are already in the input form of ``kind`` (``quantise_rows``): 16-bit rows for ``bf16``,
    e4m3 rows with their scales otherwise (python/minisgl/quant/kernels.py:562-873,1181-1331)."""
    if kind == "bf16":
        w13, w2 = weights
        return gemm_grouped(K.act_and_mul(gemm_grouped(xq, w13, tile_expert)), w2, tile_expert)
    if kind == "mxfp4":
        p13, a13, p2, a2 = weights
        aq, asc = K.silu_and_mul_quant(gemm_grouped_w4a8(xq, xsc, p13, a13, tile_expert, out_dtype))
        return gemm_grouped_w4a8(aq, asc, p2, a2, tile_expert, out_dtype)
    if kind == "fp8_channel":
        q13, s13, q2, s2 = weights
        aq, asc = K.silu_and_mul_quant(gemm_grouped_w8a8(xq, xsc, q13, s13, tile_expert, out_dtype))
        return gemm_grouped_w8a8(aq, asc, q2, s2, tile_expert, out_dtype)
    if kind == "fp8_block":
        q13, s13, q2, s2 = weights
        aq, asc = K.silu_and_mul_quant_group(K.gemm_fp8_block(xq, xsc, q13, s13, out_dtype, tile_expert=tile_expert))
        return K.gemm_fp8_block(aq, asc, q2, s2, out_dtype, tile_expert=tile_expert)
    raise ValueError(kind)


def run_experts(kind: str, xs, tile_expert, weights, out_dtype):
    """Expert MLPs of kind ``bf16 | mxfp4 | fp8_channel | fp8_block`` on 16-bit expert-sorted rows."""
    xq, xsc = quantise_rows(kind, xs)
    return run_experts_q(kind, xq, xsc, tile_expert, weights, out_dtype)


def moe_forward_quant(kind: str, x, weights, topk_w, topk_ids, expert_offset=0, counts=None):
    """align → permute → quantise → grouped GEMM → SiLU·mul + quantise → grouped GEMM → combine
    for quantised expert stacks ``weights`` of ``kind``."""
    e_local = weights[0].shape[0]
    k = topk_ids.shape[1]
    sorted_pair, pair_row, tile_expert, _meta = moe_align(topk_ids, expert_offset, e_local, counts)
    xs = _permute(x, sorted_pair, k)
    y = run_experts(kind, xs, tile_expert, weights, x.dtype)
    return _combine(y, topk_w, pair_row, x, k)
