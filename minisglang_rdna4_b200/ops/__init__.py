"""Op entry points used by layers.

A CUDA tensor is served by the hand-written sm_100a kernels in ``ops.cuda`` (which raise if
the native library is missing: there is no silent eager fallback on a GPU). A CPU tensor is
served by the fp32 PyTorch restatements in ``ops.ref``: that path is the numerics oracle and
runs the CPU plumbing configuration.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ref


def _cuda():
    from . import cuda

    return cuda


# ---------------------------------------------------------------------------- elementwise
def embedding(ids, weight, vocab_start: int = 0, vocab_len: Optional[int] = None):
    if weight.is_cuda:
        return _cuda().embedding(ids, weight, vocab_start, vocab_len)
    return ref.embedding(ids, weight, vocab_start, vocab_len)


def rms_norm(x, w, eps: float, plus_one: bool = False):
    if x.is_cuda:
        return _cuda().rms_norm(x, w, eps, plus_one)
    return ref.rms_norm(x, w, eps, plus_one)


def rms_norm_add(x, residual, w, eps: float, plus_one: bool = False):
    """``residual += x`` in place; returns ``norm(residual) * w``."""
    if x.is_cuda:
        return _cuda().rms_norm_add(x, residual, w, eps, plus_one)
    return ref.rms_norm_add(x, residual, w, eps, plus_one)


def rms_norm_quant(x, w, eps: float, residual=None, plus_one: bool = False):
    """Norm (optionally after ``residual += x``) with a per-token e4m3 producer:
    returns ``(q, scale)`` (python/minisgl/layers/norm.py:134-168)."""
    if x.is_cuda:
        return _cuda().rms_norm_quant(x, w, eps, residual, plus_one)
    y = ref.rms_norm(x, w, eps, plus_one) if residual is None else ref.rms_norm_add(x, residual, w, eps, plus_one)
    return ref.per_token_quant_fp8(y)


def per_token_quant_fp8(x):
    if x.is_cuda:
        return _cuda().per_token_quant_fp8(x)
    return ref.per_token_quant_fp8(x)


def per_group_quant_fp8(x, group: int = 128):
    if x.is_cuda:
        return _cuda().per_group_quant_fp8(x, group)
    return ref.per_group_quant_fp8(x, group)


def silu_and_mul(x):
    if x.is_cuda:
        return _cuda().act_and_mul(x, "silu")
    return ref.silu_and_mul(x)


def gelu_and_mul(x, tanh: bool = False):
    if x.is_cuda:
        return _cuda().act_and_mul(x, "gelu_tanh" if tanh else "gelu")
    return ref.gelu_and_mul(x, tanh)


def silu_and_mul_quant(x):
    """SiLU(gate)·up followed by per-token e4m3 quantisation: ``(q, scale)``."""
    if x.is_cuda:
        return _cuda().silu_and_mul_quant(x)
    return ref.per_token_quant_fp8(ref.silu_and_mul(x))


# ---------------------------------------------------------------------------- attention side
def qk_norm_rope_store(qkv, q_w, k_w, positions, cos_sin, num_q_heads: int, num_kv_heads: int,
                       head_dim: int, rotary_dim: int, eps: float, k_cache, v_cache, out_loc,
                       k_scale=None, v_scale=None, interleaved: bool = False):
    """Fused per-head QK RMSNorm + rotary embedding + KV scatter.

    ``qkv`` ``[T, (Hq + 2 Hk) * D]``. Returns the rotated queries ``[T, Hq, D]``; K and V are
    written to the paged pool at ``out_loc`` (cast or scaled to e4m3 when scales are given).
    Replaces the reference's ``qk_norm_rope`` + ``store_kv`` pair
    (python/minisgl/layers/attention.py:137-141, python/minisgl/kvcache/mha_pool.py:189-192).
    """
    if qkv.is_cuda:
        return _cuda().qk_norm_rope_store(qkv, q_w, k_w, positions, cos_sin, num_q_heads, num_kv_heads,
                                          head_dim, rotary_dim, eps, k_cache, v_cache, out_loc,
                                          k_scale, v_scale, interleaved)
    qs, ks = num_q_heads * head_dim, num_kv_heads * head_dim
    q, k, v = qkv.split([qs, ks, ks], dim=-1)
    q, k = ref.qk_norm_rope(q, k, q_w, k_w, positions, cos_sin, head_dim, rotary_dim, eps, interleaved)
    ref.store_kv(k, v, k_cache, v_cache, out_loc, k_scale, v_scale)
    return q.reshape(-1, num_q_heads, head_dim)


def q_norm_rope(q, q_w, positions, cos_sin, num_q_heads: int, head_dim: int, rotary_dim: int, eps: float,
                interleaved: bool = False):
    """Per-head RMSNorm + rotary embedding of the queries alone ``[T, Hq * D]`` → ``[T, Hq, D]``: the form a
    layer takes that reads another layer's K/V (Gemma-4's shared layers) and so has nothing to store."""
    if q.is_cuda:
        raise NotImplementedError("no kernel for the query-only norm + rotary step of a layer that shares K/V")
    dummy_k = q[:, :head_dim]
    out, _ = ref.qk_norm_rope(q, dummy_k, q_w, q_w, positions, cos_sin, head_dim, rotary_dim, eps, interleaved)
    return out.reshape(-1, num_q_heads, head_dim)


def store_kv(k, v, k_cache, v_cache, out_loc, k_scale=None, v_scale=None):
    if k.is_cuda:
        return _cuda().store_kv(k, v, k_cache, v_cache, out_loc, k_scale, v_scale)
    return ref.store_kv(k, v, k_cache, v_cache, out_loc, k_scale, v_scale)


def paged_attention(q, k_cache, v_cache, block_table, cu_q, seq_lens, scale: float, *, causal: bool = True,
                    window: int = 0, mask=None, k_scale=None, v_scale=None, max_q: int = 0,
                    max_kv: int = 0, decode: bool = False, workspace=None, splits=None, mask_window: int = 0):
    if q.is_cuda:
        return _cuda().paged_attention(q, k_cache, v_cache, block_table, cu_q, seq_lens, scale,
                                       causal=causal, window=window, mask=mask, k_scale=k_scale,
                                       v_scale=v_scale, max_q=max_q, max_kv=max_kv, decode=decode,
                                       workspace=workspace, splits=splits, mask_window=mask_window)
    return ref.paged_attention(q, k_cache, v_cache, block_table, cu_q, seq_lens, scale, causal, window,
                               mask, k_scale, v_scale, mask_window)


# ---------------------------------------------------------------------------- GEMMs
def gemm(x, w, bias=None, out_dtype: Optional[torch.dtype] = None):
    """``x @ w.T (+ bias)`` with 16-bit operands and fp32 accumulation."""
    if x.is_cuda:
        return _cuda().gemm(x, w, bias, out_dtype)
    return ref.gemm(x, w, bias, out_dtype)


def gemm_w8a8(x_q, x_scale, w_q, w_scale, out_dtype=torch.bfloat16, bias=None):
    if x_q.is_cuda:
        return _cuda().gemm_w8a8(x_q, x_scale, w_q, w_scale, out_dtype, bias)
    return ref.gemm_w8a8(x_q, x_scale, w_q, w_scale, out_dtype, bias)


def gemm_w4a8_mxfp4(x_q, x_scale, w_packed, w_sf, sf_atoms=None, out_dtype=torch.bfloat16, bias=None):
    if x_q.is_cuda:
        return _cuda().gemm_w4a8_mxfp4(x_q, x_scale, w_packed, sf_atoms, out_dtype, bias)
    return ref.gemm_w4a8_mxfp4(x_q, x_scale, w_packed, w_sf, out_dtype, bias)


def gemm_fp8_block(x_q, x_scale, w_q, w_scale, out_dtype=torch.bfloat16):
    if x_q.is_cuda:
        return _cuda().gemm_fp8_block(x_q, x_scale, w_q, w_scale, out_dtype)
    return ref.gemm_fp8_block(x_q, x_scale, w_q, w_scale, 128, out_dtype)


# ---------------------------------------------------------------------------- gated delta net
def gdn_conv1d(x, weight, conv_state, cu_q, slots, has_state, bias=None):
    if x.is_cuda:
        return _cuda().gdn_conv1d(x, weight, conv_state, cu_q, slots, has_state, bias)
    return ref.causal_conv1d(x, weight, conv_state, cu_q, slots, has_state, bias)


def mamba2_scan(xbc, dt, a_log, d_skip, dt_bias, state, cu_q, slots, has_state, heads: int, groups: int,
                head_dim: int, state_size: int, dt_min: float = 0.0):
    """Selective state-space recurrence on the rows ``xbc = [x heads ‖ B groups ‖ C groups]`` left by the
    convolution (python/minisgl/mamba2/)."""
    if xbc.is_cuda:
        return _cuda().mamba2_scan(xbc, dt, a_log, d_skip, dt_bias, state, cu_q, slots, has_state, heads, groups,
                                   head_dim, state_size, dt_min)
    t = xbc.shape[0]
    x, b, c = xbc.split([heads * head_dim, groups * state_size, groups * state_size], dim=-1)
    return ref.mamba2_scan(x.reshape(t, heads, head_dim), dt, b.reshape(t, groups, state_size),
                           c.reshape(t, groups, state_size), a_log, d_skip, dt_bias, state, cu_q, slots, has_state,
                           dt_min)


def rms_norm_gate_first(x, z, w, eps: float, group: int):
    if x.is_cuda:
        return _cuda().rms_norm_gate_first(x, z, w, eps, group)
    return ref.rms_norm_gate_first(x, z, w, eps, group)


def relu2(x):
    if x.is_cuda:
        return _cuda().relu2(x)
    return ref.relu2(x)


def gdn_recurrent(qkv, a, b, a_log, dt_bias, state, cu_q, slots, has_state, hk: int, hv: int, dk: int, dv: int):
    """Gated delta rule on the rows ``qkv = [q heads ‖ k heads ‖ v heads]`` left by the convolution."""
    if qkv.is_cuda:
        return _cuda().gdn_recurrent(qkv, a, b, a_log, dt_bias, state, cu_q, slots, has_state, hk, hv, dk, dv)
    t = qkv.shape[0]
    q, k, v = qkv.split([hk * dk, hk * dk, hv * dv], dim=-1)
    g, beta = ref.gdn_gates(a, b, a_log, dt_bias)
    return ref.gdn_recurrent(q.reshape(t, hk, dk), k.reshape(t, hk, dk), v.reshape(t, hv, dv), g, beta, state,
                             cu_q, slots, has_state)


def rms_norm_gated(x, z, w, eps: float):
    if x.is_cuda:
        return _cuda().rms_norm_gated(x, z, w, eps)
    return ref.rms_norm_gated(x, z.reshape(x.shape), w, eps)


# ---------------------------------------------------------------------------- sampling
def argmax(logits):
    if logits.is_cuda:
        return _cuda().argmax(logits)
    return logits.float().argmax(-1).to(torch.int32)


def sample(logits, temperatures, top_k=None, top_p=None, min_p=None, generator=None, uniform=None):
    if logits.is_cuda:
        return _cuda().sample(logits, temperatures, top_k, top_p, min_p, generator, uniform)
    return ref.sample(logits, temperatures, top_k, top_p, min_p, generator, uniform)


# ---------------------------------------------------------------------------- MoE
def moe_route(router_logits, top_k: int, renormalize: bool, scoring: str = "softmax", bias=None,
              scale: float = 1.0):
    if router_logits.is_cuda:
        return _cuda().moe_route(router_logits, top_k, renormalize, scoring, bias, scale)
    return ref.moe_route(router_logits, top_k, renormalize, scoring, bias, scale)


def moe_forward(x, w13, w2, topk_w, topk_ids, expert_offset: int = 0):
    if x.is_cuda:
        return _cuda().moe_forward(x, w13, w2, topk_w, topk_ids, expert_offset)
    return ref.moe_forward(x, w13, w2, topk_w, topk_ids, expert_offset)


def moe_forward_plain(x, w1, w2, topk_w, topk_ids, expert_offset: int = 0, counts=None, act: str = "relu2"):
    if x.is_cuda:
        from . import moe_kernels

        return moe_kernels.moe_forward_plain(x, w1, w2, topk_w, topk_ids, expert_offset, counts, act)
    return ref.moe_forward_plain(x, w1, w2, topk_w, topk_ids, expert_offset, act)


__all__ = [n for n in dir() if not n.startswith("_")]
