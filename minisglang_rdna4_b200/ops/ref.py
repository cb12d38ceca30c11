"""Plain PyTorch restatements of every op, computed in fp32.

These are the oracle that the CUDA kernels are tested against and the execution path of the
CPU engine (the tiny-Llama plumbing configuration runs entirely on them). Nothing here is
tuned; clarity wins.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


# ------------------------------------------------------------------------------------------
# embedding / norms / activations
# ------------------------------------------------------------------------------------------
def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0,
              vocab_len: Optional[int] = None) -> torch.Tensor:
    """``out[i] = weight[ids[i] - vocab_start]`` or zeros when the id is outside the shard
    (python/minisgl/kernel/csrc/jit/index.cu:31-96)."""
    n = weight.shape[0] if vocab_len is None else vocab_len
    local = ids.long() - vocab_start
    inside = (local >= 0) & (local < n)
    rows = weight[local.clamp(0, weight.shape[0] - 1)]
    return torch.where(inside[:, None], rows, torch.zeros_like(rows))


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, plus_one: bool = False) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    wf = w.float() + 1.0 if plus_one else w.float()
    return (xf * torch.rsqrt(var + eps) * wf).to(x.dtype)


def rms_norm_add(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                 plus_one: bool = False) -> torch.Tensor:
    """``residual += x`` in place (rounded to the storage dtype), returns norm(residual)."""
    residual.copy_((x.float() + residual.float()).to(residual.dtype))
    return rms_norm(residual, w, eps, plus_one)


def per_token_quant_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dynamic per-row e4m3: ``scale = max(amax, 1e-8) / 448``
    (python/minisgl/quant/kernels.py:1707)."""
    xf = x.float()
    amax = xf.abs().amax(-1, keepdim=True).clamp_min(1e-8)
    scale = amax / FP8_MAX
    q = (xf / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale.squeeze(-1)


def per_group_quant_fp8(x: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dynamic e4m3 with one scale per ``group`` consecutive elements of a row (1x128 groups)."""
    m, k = x.shape
    xf = x.float().view(m, k // group, group)
    amax = xf.abs().amax(-1, keepdim=True).clamp_min(1e-8)
    scale = amax / FP8_MAX
    q = (xf / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(m, k)
    return q, scale.squeeze(-1)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    gate, up = x.float().chunk(2, dim=-1)
    return (F.silu(gate) * up).to(x.dtype)


def gelu_and_mul(x: torch.Tensor, tanh: bool = False) -> torch.Tensor:
    gate, up = x.float().chunk(2, dim=-1)
    return (F.gelu(gate, approximate="tanh" if tanh else "none") * up).to(x.dtype)


# ------------------------------------------------------------------------------------------
# rotary embedding
# ------------------------------------------------------------------------------------------
def build_cos_sin_cache(rotary_dim: int, max_position: int, base: float,
                        scaling: Optional[dict] = None) -> torch.Tensor:
    """``[max_position, rotary_dim]`` float32: first half cos, second half sin. Supports the
    plain, linear, llama3 and yarn frequency schedules
    (python/minisgl/layers/rotary.py:13-262)."""
    half = rotary_dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float64) * 2 / rotary_dim))
    mscale = 1.0
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            inv_freq = inv_freq / factor
        elif kind == "llama3":
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = ((orig / wavelen) - low) / (high - low)
            scaled = torch.where(
                wavelen > orig / low, inv_freq / factor,
                torch.where(wavelen < orig / high, inv_freq,
                            (1 - smooth) * inv_freq / factor + smooth * inv_freq))
            inv_freq = scaled
        elif kind == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", max_position))
            beta_fast = float(scaling.get("beta_fast", 32.0))
            beta_slow = float(scaling.get("beta_slow", 1.0))

            def corr_dim(rot):
                return rotary_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(base))

            lo = max(math.floor(corr_dim(beta_fast)), 0)
            hi = min(math.ceil(corr_dim(beta_slow)), half - 1)
            ramp = ((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            mask = 1.0 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask
            def yarn_mscale(m: float = 1.0) -> float:
                return 0.1 * m * math.log(factor) + 1.0 if factor > 1 else 1.0

            if scaling.get("attention_factor"):
                mscale = float(scaling["attention_factor"])
            elif scaling.get("mscale") and scaling.get("mscale_all_dim"):
                # DeepSeek-style YaRN: the table carries the ratio of the two magnitude factors (the softmax
                # scale of the attention layer carries mscale_all_dim squared)
                mscale = yarn_mscale(float(scaling["mscale"])) / yarn_mscale(float(scaling["mscale_all_dim"]))
            else:
                mscale = yarn_mscale()
        elif kind == "proportional":
            # Gemma-4 global layers: the first partial_rotary_factor of the pairs (i, i + dim/2) rotate with
            # the frequencies of the full width, the others keep angle zero
            angles = int(float(scaling.get("partial_rotary_factor", 1.0)) * rotary_dim // 2)
            inv_freq = torch.where(torch.arange(half) < angles, inv_freq, torch.zeros_like(inv_freq)) / factor
        elif kind in ("default", "dynamic", None):
            pass
        else:
            raise ValueError(f"unsupported rope scaling {kind!r}")
    t = torch.arange(max_position, dtype=torch.float64)
    freqs = torch.outer(t, inv_freq)
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).float()


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    # x [T, H, rot]; cos/sin [T, rot/2]
    if interleaved:
        x1, x2 = x[..., 0::2], x[..., 1::2]
        o1 = x1 * cos[:, None] - x2 * sin[:, None]
        o2 = x2 * cos[:, None] + x1 * sin[:, None]
        return torch.stack([o1, o2], dim=-1).flatten(-2)
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos[:, None] - x2 * sin[:, None], x2 * cos[:, None] + x1 * sin[:, None]], dim=-1)


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_w: Optional[torch.Tensor],
                 k_w: Optional[torch.Tensor], positions: torch.Tensor, cos_sin: torch.Tensor,
                 head_dim: int, rotary_dim: int, eps: float, interleaved: bool = False,
                 plus_one: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-head RMSNorm of q and k (when weights are given) followed by rotary embedding on the
    first ``rotary_dim`` dims. ``q`` ``[T, Hq*D]``, ``k`` ``[T, Hk*D]``; returns new tensors
    (python/minisgl/layers/attention.py:100-141)."""
    t = q.shape[0]
    qf = q.float().view(t, -1, head_dim)
    kf = k.float().view(t, -1, head_dim)
    if q_w is not None:
        wq = q_w.float() + (1.0 if plus_one else 0.0)
        wk = k_w.float() + (1.0 if plus_one else 0.0)
        qf = qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + eps) * wq
        kf = kf * torch.rsqrt(kf.pow(2).mean(-1, keepdim=True) + eps) * wk
        # the kernels round the normed value to the storage dtype before rotating
        qf = qf.to(q.dtype).float()
        kf = kf.to(k.dtype).float()
    cs = cos_sin[positions.long()]
    cos, sin = cs[:, : rotary_dim // 2], cs[:, rotary_dim // 2 :]
    q_rot = _rotate(qf[..., :rotary_dim], cos, sin, interleaved)
    k_rot = _rotate(kf[..., :rotary_dim], cos, sin, interleaved)
    qo = torch.cat([q_rot, qf[..., rotary_dim:]], dim=-1).to(q.dtype).view(t, -1)
    ko = torch.cat([k_rot, kf[..., rotary_dim:]], dim=-1).to(k.dtype).view(t, -1)
    return qo, ko


# ------------------------------------------------------------------------------------------
# KV store + paged attention
# ------------------------------------------------------------------------------------------
def store_kv(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             out_loc: torch.Tensor, k_scale: Optional[torch.Tensor] = None,
             v_scale: Optional[torch.Tensor] = None) -> None:
    """Scatter rows into the paged pool ``[pages, heads, page_size, dim]``; with scales the
    value is divided by the per-head descale and stored as e4m3
    (python/minisgl/kvcache/mha_pool.py:169-193)."""
    ps = k_cache.shape[2]
    heads, dim = k_cache.shape[1], k_cache.shape[3]
    t = out_loc.numel()
    kk = k.reshape(t, heads, dim)
    vv = v.reshape(t, heads, dim)
    loc = out_loc.long()
    page, off = loc // ps, loc % ps
    if k_scale is not None:
        kq = (kk.float() / k_scale.float()[None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(k_cache.dtype)
        vq = (vv.float() / v_scale.float()[None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(v_cache.dtype)
    else:
        kq, vq = kk.to(k_cache.dtype), vv.to(v_cache.dtype)
    k_cache[page, :, off] = kq
    v_cache[page, :, off] = vq


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor,
                    scale: float, causal: bool = True, window: int = 0,
                    mask: Optional[torch.Tensor] = None, k_scale: Optional[torch.Tensor] = None,
                    v_scale: Optional[torch.Tensor] = None, mask_window: int = 0) -> torch.Tensor:
    """Attention of packed queries over paged KV.

    ``q`` ``[T, Hq, D]``; request ``b`` owns rows ``cu_q[b]:cu_q[b+1]`` which are the LAST
    ``q_len`` positions of a sequence of ``seq_lens[b]`` tokens whose KV sits in pages
    ``block_table[b]``. ``causal``: row at absolute position p sees kv positions <= p.
    ``window`` > 0 additionally hides positions <= p - window. ``mask`` is an additive
    ``[T, >=max_kv]`` float bias (tree verification); when given it replaces the causal rule.
    With ``mask_window`` > 0 the mask is ``[T, mask_window]`` and covers only the last
    ``mask_window`` KV positions of each request; earlier positions are visible to every row
    (of a sliding-window layer: to the rows that have them inside their window).
    """
    t, hq, d = q.shape
    hk, ps = k_cache.shape[1], k_cache.shape[2]
    group = hq // hk
    out = torch.zeros_like(q, dtype=torch.float32)
    cu = cu_q.tolist()
    lens = seq_lens.tolist()
    for b in range(len(lens)):
        qs, qe, kv_len = cu[b], cu[b + 1], lens[b]
        q_len = qe - qs
        if q_len == 0 or kv_len == 0:
            continue
        n_pages = -(-kv_len // ps)
        pages = block_table[b, :n_pages].long()
        kk = k_cache[pages].float().permute(1, 0, 2, 3).reshape(hk, n_pages * ps, d)[:, :kv_len]
        vv = v_cache[pages].float().permute(1, 0, 2, 3).reshape(hk, n_pages * ps, d)[:, :kv_len]
        if k_scale is not None:
            kk = kk * k_scale.float()[:, None, None]
            vv = vv * v_scale.float()[:, None, None]
        qq = q[qs:qe].float().permute(1, 0, 2).reshape(hk, group * q_len, d)  # head h -> kv h//group
        qq = q[qs:qe].float().view(q_len, hk, group, d).permute(1, 2, 0, 3)    # [hk, g, q, d]
        s = torch.einsum("hgqd,hkd->hgqk", qq, kk) * scale
        q_pos = torch.arange(kv_len - q_len, kv_len, device=q.device)[:, None]
        k_pos = torch.arange(kv_len, device=q.device)[None, :]
        if mask is not None and mask_window:
            w = min(mask_window, kv_len)
            full = torch.zeros(q_len, kv_len, dtype=torch.float32, device=q.device)
            full[:, kv_len - w:] = mask[qs:qe, mask_window - w:mask_window].float()
            if window and window > 0 and kv_len > w:
                early = (k_pos <= q_pos - window) & (k_pos < kv_len - w)
                full = full.masked_fill(early, float("-inf"))
            s = s + full[None, None]
        elif mask is not None:
            s = s + mask[qs:qe, :kv_len].float()[None, None]
        else:
            if causal:
                s = s.masked_fill((k_pos > q_pos)[None, None], float("-inf"))
            if window and window > 0:
                s = s.masked_fill((k_pos <= q_pos - window)[None, None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)
        o = torch.einsum("hgqk,hkd->hgqd", p, vv)  # [hk, g, q, d]
        out[qs:qe] = o.permute(2, 0, 1, 3).reshape(q_len, hq, d)
    return out.to(q.dtype)


def mla_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, rows: torch.Tensor, block_table: torch.Tensor,
                  cu_q: torch.Tensor, seq_lens: torch.Tensor, scale: float, lora_rank: int) -> torch.Tensor:
    """Absorbed latent attention over a paged pool of ``[latent ‖ rotary key]`` rows.

    ``q_lat`` ``[T, H, lora]`` (queries already multiplied by the key half of ``kv_b_proj``), ``q_rot``
    ``[T, H, rope]``, ``rows`` ``[pages, page_size, lora + rope]``. Every head attends to the same
    single key per position: score = ``q_lat . latent + q_rot . k_rot``; causal; the result is the
    softmax-weighted sum of the latents ``[T, H, lora]`` (the value half of ``kv_b_proj`` is applied by
    the caller). Written with tensor ops that run on either device
    (python/minisgl/attention/mla.py:99-161)."""
    t, h, _ = q_lat.shape
    ps = rows.shape[1]
    out = torch.zeros((t, h, lora_rank), dtype=torch.float32, device=q_lat.device)
    cu = cu_q.tolist()
    lens = seq_lens.tolist()
    for b in range(len(lens)):
        qs, qe, kv_len = cu[b], cu[b + 1], lens[b]
        q_len = qe - qs
        if q_len == 0 or kv_len == 0:
            continue
        n_pages = -(-kv_len // ps)
        kv = rows[block_table[b, :n_pages].long()].reshape(n_pages * ps, -1)[:kv_len].float()
        lat, rot = kv[:, :lora_rank], kv[:, lora_rank:]
        s = (torch.einsum("qhl,kl->hqk", q_lat[qs:qe].float(), lat)
             + torch.einsum("qhr,kr->hqk", q_rot[qs:qe].float(), rot)) * scale
        q_pos = torch.arange(kv_len - q_len, kv_len, device=s.device)[:, None]
        k_pos = torch.arange(kv_len, device=s.device)[None, :]
        s = s.masked_fill((k_pos > q_pos)[None], float("-inf"))
        out[qs:qe] = torch.einsum("hqk,kl->qhl", torch.softmax(s, dim=-1), lat)
    return out.to(q_lat.dtype)


# ------------------------------------------------------------------------------------------
# quantised GEMMs (reference dequantises the weight and multiplies in fp32)
# ------------------------------------------------------------------------------------------
def e8m0_to_float(s: torch.Tensor) -> torch.Tensor:
    """UE8M0 byte → ``2^(s-127)``; 0xFF is NaN (python/minisgl/quant/mxfp4.py:72-95)."""
    out = torch.pow(2.0, s.to(torch.float32) - 127.0)
    return torch.where(s == 255, torch.full_like(out, float("nan")), out)


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """``[N, K/2]`` bytes → ``[N, K]`` float32; the low nibble is the even k."""
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=packed.device)
    b = packed.to(torch.uint8)
    lo, hi = (b & 0xF).long(), (b >> 4).long()
    return torch.stack([lut[lo], lut[hi]], dim=-1).flatten(-2)


def dequant_mxfp4(packed: torch.Tensor, scales: torch.Tensor, group: int = 32) -> torch.Tensor:
    w = unpack_e2m1(packed)
    return w * e8m0_to_float(scales).repeat_interleave(group, dim=-1)


def dequant_nvfp4(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor,
                  group: int = 16) -> torch.Tensor:
    """e2m1 × e4m3 block scale × per-channel fp32 multiplier
    (python/minisgl/quant/nvfp4.py:81-179)."""
    w = unpack_e2m1(packed)
    sf = scales.to(torch.float32).repeat_interleave(group, dim=-1)
    return w * sf * global_scale.float().reshape(-1, 1)


def gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
         out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or x.dtype)


def gemm_w8a8(x_q: torch.Tensor, x_scale: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor,
              out_dtype: torch.dtype = torch.bfloat16, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-token activation scale × per-channel weight scale."""
    y = (x_q.float() @ w_q.float().t()) * x_scale.float()[:, None] * w_scale.float().reshape(1, -1)
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)


def gemm_w4a8_mxfp4(x_q: torch.Tensor, x_scale: torch.Tensor, w_packed: torch.Tensor,
                    w_sf: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                    bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    w = dequant_mxfp4(w_packed, w_sf)
    y = (x_q.float() @ w.t()) * x_scale.float()[:, None]
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype)


def gemm_fp8_block(x_q: torch.Tensor, x_scale: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor,
                   block: int = 128, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """1x128 activation groups × 128x128 weight blocks."""
    m, k = x_q.shape
    n = w_q.shape[0]
    xs = x_scale.float().repeat_interleave(block, dim=-1)[:, :k]
    ws = w_scale.float().repeat_interleave(block, 0).repeat_interleave(block, 1)[:n, :k]
    return ((x_q.float() * xs) @ (w_q.float() * ws).t()).to(out_dtype)


# ------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperatures: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], min_p: Optional[torch.Tensor],
           generator: Optional[torch.Generator] = None,
           uniform: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(logits / max(T, 1e-6))`` → min-p floor → top-k → top-p over the surviving
    sorted mass → renormalise → draw; rows with T == 0 take the argmax
    (python/minisgl/engine/sample.py:108-142). ``uniform`` ``[bs]`` gives the random numbers
    explicitly (inverse-CDF draw over the sorted distribution) so a kernel can be compared."""
    lf = logits.float()
    greedy = temperatures <= 0
    arg = lf.argmax(-1)
    if bool(greedy.all()):
        return arg.to(torch.int32)
    probs = torch.softmax(lf / temperatures.clamp_min(1e-6)[:, None], dim=-1)
    if min_p is not None:
        floor = probs.amax(-1, keepdim=True) * min_p[:, None]
        probs = torch.where(probs < floor, torch.zeros_like(probs), probs)
    sorted_p, sorted_i = probs.sort(-1, descending=True)
    if top_k is not None:
        ranks = torch.arange(probs.shape[-1], device=probs.device)[None, :]
        kk = torch.where(top_k <= 0, torch.full_like(top_k, probs.shape[-1]), top_k)
        sorted_p = torch.where(ranks >= kk[:, None], torch.zeros_like(sorted_p), sorted_p)
    if top_p is not None:
        csum = sorted_p.cumsum(-1)
        sorted_p = torch.where(csum - sorted_p > top_p[:, None], torch.zeros_like(sorted_p), sorted_p)
    sorted_p = sorted_p / sorted_p.sum(-1, keepdim=True)
    if uniform is not None:
        cdf = sorted_p.cumsum(-1)
        pick = (cdf < uniform[:, None]).sum(-1).clamp_max(probs.shape[-1] - 1)
    else:
        pick = torch.multinomial(sorted_p, 1, generator=generator).squeeze(-1)
    drawn = sorted_i.gather(-1, pick[:, None]).squeeze(-1)
    return torch.where(greedy, arg, drawn).to(torch.int32)


# ------------------------------------------------------------------------------------------
# mixture of experts
# ------------------------------------------------------------------------------------------
def moe_route(router_logits: torch.Tensor, top_k: int, renormalize: bool, scoring: str = "softmax",
              bias: Optional[torch.Tensor] = None, scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k routing weights and expert ids ``[T, top_k]``."""
    g = router_logits.float()
    scores = torch.softmax(g, dim=-1) if scoring == "softmax" else torch.sigmoid(g)
    pick = scores + bias.float() if bias is not None else scores
    _, ids = pick.topk(top_k, dim=-1)
    w = scores.gather(-1, ids)
    if renormalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return (w * scale).float(), ids.to(torch.int32)


def moe_route_grouped(router_logits: torch.Tensor, top_k: int, renormalize: bool, scoring: str,
                      bias: Optional[torch.Tensor], scale: float, n_group: int, topk_group: int
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group-limited routing (DeepSeek-V3 / GLM-4 MoE): experts are split into ``n_group`` groups,
    a group's score is the sum of its two best choice scores, only the best ``topk_group`` groups
    stay eligible, then top-k over the eligible experts; weights are the un-biased scores.
    Without a selection bias (DeepSeek-V2's ``group_limited_greedy``) a group's score is its best
    expert's score."""
    g = router_logits.float()
    scores = torch.softmax(g, dim=-1) if scoring == "softmax" else torch.sigmoid(g)
    choice = scores + bias.float() if bias is not None else scores
    t, e = choice.shape
    grouped = choice.view(t, n_group, e // n_group)
    group_scores = grouped.max(-1)[0] if bias is None else grouped.topk(2, dim=-1)[0].sum(-1)
    keep = torch.zeros_like(group_scores)
    keep.scatter_(1, group_scores.topk(topk_group, dim=-1, sorted=False)[1], 1.0)
    mask = keep[:, :, None].expand(t, n_group, e // n_group).reshape(t, e).bool()
    _, ids = choice.masked_fill(~mask, 0.0).topk(top_k, dim=-1)
    w = scores.gather(-1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return (w * scale).float(), ids.to(torch.int32)


def moe_forward(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                topk_ids: torch.Tensor, expert_offset: int = 0, act: str = "silu") -> torch.Tensor:
    """``sum_k w_k * down_e(act(gate_e x) * up_e x)`` over the experts held locally
    (``w13`` ``[E_local, 2I, H]``, ``w2`` ``[E_local, H, I]``); ids outside the local range
    contribute nothing. ``act``: ``silu`` or ``gelu_pytorch_tanh`` (Gemma-4 experts)."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    e_local = w13.shape[0]
    xf = x.float()
    for e in range(e_local):
        sel = (topk_ids == e + expert_offset)
        rows = sel.any(-1).nonzero().squeeze(-1)
        if rows.numel() == 0:
            continue
        wt = (topk_w * sel).sum(-1)[rows]
        hcur = xf[rows] @ w13[e].float().t()
        gate, up = hcur.chunk(2, dim=-1)
        g_act = F.silu(gate) if act == "silu" else F.gelu(gate, approximate="tanh")
        hid = (g_act * up).to(x.dtype).float()
        out[rows] += (hid @ w2[e].float().t()) * wt[:, None]
    return out.to(x.dtype)


def moe_forward_plain(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                      topk_ids: torch.Tensor, expert_offset: int = 0, act: str = "relu2") -> torch.Tensor:
    """``sum_k w_k * down_e(act(up_e x))`` for non-gated experts (``w1 [E, I, H]``, ``w2 [E, H, I]``)."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(w1.shape[0]):
        sel = (topk_ids == e + expert_offset)
        rows = sel.any(-1).nonzero().squeeze(-1)
        if rows.numel() == 0:
            continue
        wt = (topk_w * sel).sum(-1)[rows]
        hcur = relu2((xf[rows] @ w1[e].float().t()).to(x.dtype)).float()
        out[rows] += (hcur @ w2[e].float().t()) * wt[:, None]
    return out.to(x.dtype)


# ------------------------------------------------------------------------------------------
# gated delta net (linear attention with a recurrent state)
# ------------------------------------------------------------------------------------------
def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, conv_state: torch.Tensor, cu_q: torch.Tensor,
                  slots: torch.Tensor, has_state: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Depthwise causal convolution + SiLU over packed sequences.

    ``x [T, C]`` holds the rows of B sequences (``cu_q [B+1]``); ``weight [C, Kw]``;
    ``conv_state [slots, C, Kw-1]`` keeps the last ``Kw-1`` inputs of every sequence and is
    updated in place (a sequence with ``has_state == 0`` starts from zeros). Returns ``[T, C]``
    (python/minisgl/gdn/layer.py:346-420 causal_conv1d_fwd / _update)."""
    out = torch.empty_like(x)
    kw = weight.shape[1]
    wf = weight.float()
    for b in range(cu_q.numel() - 1):
        lo, hi = int(cu_q[b]), int(cu_q[b + 1])
        slot = int(slots[b])
        hist = conv_state[slot].float().t() if int(has_state[b]) else x.new_zeros((kw - 1, x.shape[1])).float()
        seq = torch.cat([hist, x[lo:hi].float()])                    # [Kw-1 + n, C]
        n = hi - lo
        acc = torch.zeros((n, x.shape[1]))
        for j in range(kw):
            acc += seq[j:j + n] * wf[:, j]
        if bias is not None:
            acc += bias.float()
        out[lo:hi] = F.silu(acc).to(x.dtype)
        conv_state[slot] = seq[-(kw - 1):].t().to(conv_state.dtype)
    return out


def gdn_gates(a: torch.Tensor, b: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor):
    """Per (token, value head): log-decay ``g = -exp(A_log) * softplus(a + dt_bias)`` and write
    strength ``beta = sigmoid(b)``."""
    g = -a_log.float().exp() * F.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


def gdn_recurrent(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                  state: torch.Tensor, cu_q: torch.Tensor, slots: torch.Tensor, has_state: torch.Tensor
                  ) -> torch.Tensor:
    """Gated delta rule, token by token (the recurrent form).

    ``q, k [T, Hk, Dk]`` (L2-normalised here, q scaled by ``Dk ** -0.5``; key heads are shared by
    ``Hv / Hk`` value heads), ``v [T, Hv, Dv]``, ``g, beta [T, Hv]``, ``state [slots, Hv, Dk, Dv]``
    fp32, updated in place. Per token: ``S *= exp(g)``; ``delta = (v - S^T k) * beta``;
    ``S += k (x) delta``; ``out = S^T q``. Returns ``[T, Hv, Dv]``
    (python/minisgl/gdn/layer.py:421-760 gdn_prefill / gdn_decode)."""
    t, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    rep = hv // hk
    qf = q.float()
    kf = k.float()
    qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    qf = qf.repeat_interleave(rep, dim=1)
    kf = kf.repeat_interleave(rep, dim=1)
    out = torch.empty((t, hv, dv), dtype=torch.float32)
    for bi in range(cu_q.numel() - 1):
        lo, hi = int(cu_q[bi]), int(cu_q[bi + 1])
        slot = int(slots[bi])
        s = state[slot].float().clone() if int(has_state[bi]) else torch.zeros((hv, dk, dv))
        for i in range(lo, hi):
            s = s * g[i].float().exp()[:, None, None]
            kv = (s * kf[i][:, :, None]).sum(1)                      # [Hv, Dv]
            delta = (v[i].float() - kv) * beta[i].float()[:, None]
            s = s + kf[i][:, :, None] * delta[:, None, :]
            out[i] = (s * qf[i][:, :, None]).sum(1)
        state[slot] = s
    return out.to(v.dtype)


def mamba2_scan(x: torch.Tensor, dt: torch.Tensor, b: torch.Tensor, c: torch.Tensor, a_log: torch.Tensor,
                d_skip: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
                slots: torch.Tensor, has_state: torch.Tensor, dt_min: float = 0.0) -> torch.Tensor:
    """Selective state-space recurrence of a Mamba-2 mixer, token by token.

    ``x [T, H, P]`` (after the convolution), ``dt [T, H]`` raw step sizes, ``b, c [T, G, N]`` (a group
    of ``H / G`` heads shares one B and C), ``a_log, d_skip, dt_bias [H]``, ``state [slots, H, P, N]``
    fp32, updated in place (a sequence with ``has_state == 0`` starts from zeros). Per token and head:
    ``dt' = max(softplus(dt + dt_bias), dt_min)``; ``S = S * exp(-exp(a_log) dt') + dt' x (x) B``;
    ``y = S C + d_skip x``. Returns ``[T, H, P]``."""
    t, h, p = x.shape
    g = b.shape[1]
    rep = h // g
    out = torch.empty((t, h, p), dtype=torch.float32)
    a = -a_log.float().exp()
    for s_i in range(cu_q.numel() - 1):
        lo, hi = int(cu_q[s_i]), int(cu_q[s_i + 1])
        slot = int(slots[s_i])
        st = state[slot].float().clone() if int(has_state[s_i]) else torch.zeros_like(state[slot], dtype=torch.float32)
        for i in range(lo, hi):
            step = torch.clamp(F.softplus(dt[i].float() + dt_bias.float()), min=dt_min)          # [H]
            bi = b[i].float().repeat_interleave(rep, dim=0)                                         # [H, N]
            ci = c[i].float().repeat_interleave(rep, dim=0)
            xi = x[i].float()                                                                       # [H, P]
            st = st * torch.exp(step * a)[:, None, None] + (step[:, None] * xi)[:, :, None] * bi[:, None, :]
            out[i] = torch.einsum("hpn,hn->hp", st, ci) + d_skip.float()[:, None] * xi
        state[slot] = st.to(state.dtype)
    return out.to(x.dtype)


def rms_norm_gate_first(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, group: int) -> torch.Tensor:
    """``w * norm_g(x * silu(z))`` where the RMS is taken over groups of ``group`` consecutive
    channels (the gate comes before the norm: Mamba-2 / Zamba-2 / Nemotron-H mixers)."""
    y = x.float() * F.silu(z.float())
    shape = y.shape
    yg = y.view(*shape[:-1], shape[-1] // group, group)
    yg = yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + eps)
    return (w.float() * yg.view(shape).to(x.dtype).float()).to(x.dtype)


def relu2(x: torch.Tensor) -> torch.Tensor:
    """Squared ReLU (the non-gated MLP activation of the Nemotron-H family)."""
    r = torch.relu(x.float())
    return (r * r).to(x.dtype)


def rms_norm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``norm(x) * w * silu(z)`` over the last dimension (the norm comes before the gate)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (w.float() * y.to(x.dtype).float()) * F.silu(z.float())
    return y.to(x.dtype)
