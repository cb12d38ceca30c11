"""NVFP4 codec: e2m1 elements, one e4m3 scale per 16 K elements, one fp32 scale per tensor
or channel.

Two producers disagree on the direction of the global scale
(python/minisgl/quant/nvfp4.py:68-69,81-130): compressed-tensors stores
``weight_global_scale = 448*6/amax`` (the value is DIVIDED out on dequantisation) while
ModelOpt stores ``weight_scale_2 = amax/(448*6)`` (MULTIPLIED). Both are normalised here to a
per-channel multiplier ``(N,)``.
"""
from __future__ import annotations

from typing import Tuple

import torch

from ..ops.ref import dequant_nvfp4, unpack_e2m1
from .mxfp4 import quantize_e2m1

GROUP = 16


def normalise_global_scale(value: torch.Tensor, n_out: int, divides: bool) -> torch.Tensor:
    v = value.float().reshape(-1)
    v = 1.0 / v if divides else v
    if v.numel() == 1:
        v = v.expand(n_out)
    assert v.numel() == n_out
    return v.contiguous()


def quantize_nvfp4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(N, K)`` → ``(packed, block scales e4m3 (N, K/16), global multiplier (N,))``."""
    n, k = w.shape
    g = w.float().view(n, k // GROUP, GROUP)
    amax_t = w.float().abs().amax().clamp_min(1e-12)
    glob = amax_t / (448.0 * 6.0)
    blk = (g.abs().amax(-1) / 6.0 / glob).clamp(max=448.0).to(torch.float8_e4m3fn)
    denom = (blk.float() * glob).clamp_min(1e-30)
    codes = quantize_e2m1(g / denom[..., None]).view(n, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, blk, glob.expand(n).contiguous()


__all__ = ["GROUP", "normalise_global_scale", "quantize_nvfp4", "dequant_nvfp4", "unpack_e2m1"]
