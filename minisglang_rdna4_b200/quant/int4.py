"""Group-wise int4 checkpoint layouts (AWQ, GPTQ, compressed-tensors pack-quantized) →
one canonical form: ``codes (N, K) uint8 in 0..15``, ``scales (N, K/g) f32``,
``zeros (N, K/g) f32`` with ``w = (code - zero) * scale``.

Layout facts (python/minisgl/quant/kernels.py:22,255-346, quant/method.py:143-244,408-445):
* AWQ ``qweight (K, N/8) i32`` packs 8 output channels per word in the order
  ``[0,4,1,5,2,6,3,7]``; ``qzeros (K/g, N/8)`` likewise; ``scales (K/g, N)``.
* GPTQ ``qweight (K/8, N) i32`` packs 8 consecutive k in natural order; ``qzeros (K/g, N/8)``
  stores ``zero - 1``.
* compressed-tensors ``weight_packed (N, K/8) i32`` natural order along K; nibbles are
  either offset-binary (uint4b8: code 8 is zero) or two's complement. The convention is
  detected from the data: real weight distributions peak at zero, so the zero code is by far
  the most frequent of {0, 8}.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

AWQ_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)
_AWQ_REVERSE = tuple(AWQ_ORDER.index(i) for i in range(8))  # position of channel i in the word


def _unpack_words(words: torch.Tensor) -> torch.Tensor:
    """int32 ``(..., W)`` → uint8 ``(..., W, 8)`` nibbles, lowest first."""
    shifts = torch.arange(0, 32, 4, device=words.device, dtype=torch.int32)
    return ((words.to(torch.int32)[..., None] >> shifts) & 0xF).to(torch.uint8)


def awq_to_canonical(qweight: torch.Tensor, scales: torch.Tensor, qzeros: Optional[torch.Tensor],
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    k, n8 = qweight.shape
    n = n8 * 8
    rev = torch.tensor(_AWQ_REVERSE, device=qweight.device)
    codes = _unpack_words(qweight)[..., rev].reshape(k, n)          # (K, N)
    if qzeros is not None:
        zeros = _unpack_words(qzeros)[..., rev].reshape(qzeros.shape[0], n).float()
    else:
        zeros = torch.full((scales.shape[0], n), 8.0, device=qweight.device)
    return codes.t().contiguous(), scales.float().t().contiguous(), zeros.t().contiguous()


def gptq_to_canonical(qweight: torch.Tensor, scales: torch.Tensor, qzeros: Optional[torch.Tensor],
                      symmetric: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    k8, n = qweight.shape
    codes = _unpack_words(qweight.t().contiguous()).reshape(n, k8 * 8)  # (N, K)
    if qzeros is not None and not symmetric:
        zeros = _unpack_words(qzeros).reshape(qzeros.shape[0], n).float() + 1.0
    else:
        zeros = torch.full((scales.shape[0], n), 8.0, device=qweight.device)
    return codes.contiguous(), scales.float().t().contiguous(), zeros.t().contiguous()


def detect_ct_sign_convention(weight_packed: torch.Tensor, max_words: int = 65536,
                              margin: float = 1e-3) -> str:
    """``"offset"`` (uint4b8) or ``"twos"``; raises when the sample is inconclusive."""
    flat = weight_packed.reshape(-1)
    if flat.numel() > max_words:
        step = flat.numel() // max_words
        flat = flat[::step][:max_words]
    nib = _unpack_words(flat).reshape(-1)
    total = max(nib.numel(), 1)
    f8 = float((nib == 8).sum()) / total
    f0 = float((nib == 0).sum()) / total
    if abs(f8 - f0) < margin:
        raise ValueError(f"int4 sign convention is ambiguous (p[8]={f8:.4f}, p[0]={f0:.4f})")
    return "offset" if f8 > f0 else "twos"


def ct_to_canonical(weight_packed: torch.Tensor, weight_scale: torch.Tensor,
                    weight_zero_point: Optional[torch.Tensor], convention: Optional[str] = None,
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    n, k8 = weight_packed.shape
    codes = _unpack_words(weight_packed).reshape(n, k8 * 8)
    convention = convention or detect_ct_sign_convention(weight_packed)
    if convention == "twos":
        codes = codes ^ 0x8  # two's complement → offset binary (XOR 0x88 on a byte of two nibbles)
    scales = weight_scale.float()
    if weight_zero_point is not None:
        zp = _unpack_words(weight_zero_point.t().contiguous()).reshape(weight_zero_point.shape[1], -1)
        zeros = zp.t()[:n].float()
        if convention == "twos":
            zeros = (zeros.to(torch.uint8) ^ 0x8).float()
    else:
        zeros = torch.full_like(scales, 8.0)
    return codes.contiguous(), scales.contiguous(), zeros.contiguous()


def dequant_int4(codes: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor) -> torch.Tensor:
    n, k = codes.shape
    g = k // scales.shape[1]
    return (codes.float() - zeros.repeat_interleave(g, 1)) * scales.repeat_interleave(g, 1)


def quantize_int4(w: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Symmetric reference quantiser (tests and dummy weights): zero code 8."""
    n, k = w.shape
    g = w.float().view(n, k // group, group)
    scale = (g.abs().amax(-1) / 7.0).clamp_min(1e-8)
    codes = (torch.round(g / scale[..., None]).clamp(-8, 7) + 8).to(torch.uint8).view(n, k)
    return codes, scale, torch.full_like(scale, 8.0)


def pack_awq(codes: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor):
    """Canonical → AWQ tensors (test helper)."""
    n, k = codes.shape
    order = torch.tensor(AWQ_ORDER, device=codes.device)
    shifts = torch.arange(0, 32, 4, device=codes.device, dtype=torch.int64)
    cw = codes.t().reshape(k, n // 8, 8)[..., order].to(torch.int64)
    qweight = (cw << shifts).sum(-1)
    zw = zeros.t().to(torch.uint8).reshape(-1, n // 8, 8)[..., order].to(torch.int64)
    qzeros = (zw << shifts).sum(-1)
    to_i32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    return to_i32(qweight), scales.t().contiguous().half(), to_i32(qzeros)


def pack_gptq(codes: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor):
    n, k = codes.shape
    shifts = torch.arange(0, 32, 4, device=codes.device, dtype=torch.int64)
    qweight = (codes.reshape(n, k // 8, 8).to(torch.int64) << shifts).sum(-1).t().contiguous()
    zw = (zeros.t() - 1).to(torch.uint8).reshape(-1, n // 8, 8).to(torch.int64)
    qzeros = (zw << shifts).sum(-1)
    to_i32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)
    return to_i32(qweight), scales.t().contiguous().half(), to_i32(qzeros)


def pack_ct(codes: torch.Tensor, scales: torch.Tensor, twos: bool = False):
    n, k = codes.shape
    c = (codes ^ 0x8) if twos else codes
    shifts = torch.arange(0, 32, 4, device=codes.device, dtype=torch.int64)
    packed = (c.reshape(n, k // 8, 8).to(torch.int64) << shifts).sum(-1)
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return packed, scales.half()
