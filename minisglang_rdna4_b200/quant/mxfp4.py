"""MXFP4 codec: e2m1 elements with one UE8M0 scale per 32 consecutive K elements.

Checkpoint layout (compressed-tensors ``mxfp4-pack-quantized``;
python/minisgl/quant/mxfp4.py:37-52,72-95,262-275): ``weight_packed (N, K/2) u8`` with the
low nibble holding the even k, ``weight_scale (N, K/32) u8`` meaning ``2^(s-127)``.

Kernel layout of the scales ("sf atoms"): the block-scaled tensor-core instruction reads
scale factors from tensor memory in groups of 128 rows x 4 K-blocks laid out as
``[32 (row % 32), 4 (row // 32), 4 (k-block)]`` bytes, so the weights' scales are stored as
``[N/128, K/128, 32, 4, 4]`` and one 512-byte atom is copied per (row tile, K tile).
"""
from __future__ import annotations

from typing import Tuple

import torch

from ..ops.ref import E2M1_VALUES, dequant_mxfp4, e8m0_to_float, unpack_e2m1

GROUP = 32
_E2M1_POS = torch.tensor(E2M1_VALUES[:8])
# decision thresholds between consecutive positive e2m1 values, ties to even mantissa
_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def quantize_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even float → e2m1 code (uint8 in 0..15), saturating at ±6."""
    ax = x.abs().float()
    bounds = _BOUNDS.to(x.device)
    idx = torch.bucketize(ax, bounds, right=False)  # ax == bound goes to the lower bucket
    # ties: 0.25→0 (even), 0.75→1.0, 1.25→1.0, 1.75→2.0, 2.5→2, 3.5→4, 5→4
    tie_up = torch.tensor([False, True, False, True, False, True, False], device=x.device)
    which = idx.clamp_max(6)
    at_tie = ax == bounds[which]
    idx = torch.where(at_tie & tie_up[which], idx + 1, idx).clamp_max(7)
    sign = (x < 0) | ((x == 0) & torch.signbit(x))
    return (idx + 8 * sign.long()).to(torch.uint8)


def quantize_mxfp4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(N, K)`` float → ``(packed (N, K/2) u8, scales (N, K/32) u8)``; the shared exponent
    is ``floor(log2(amax)) - 2`` (the OCP MX rule for an element type with emax = 2)."""
    n, k = w.shape
    assert k % GROUP == 0
    g = w.float().view(n, k // GROUP, GROUP)
    amax = g.abs().amax(-1)
    exp = torch.floor(torch.log2(amax.clamp_min(2.0 ** -126))) - 2
    exp = exp.clamp(-127, 127)
    scale = torch.pow(2.0, exp)
    codes = quantize_e2m1(g / scale[..., None]).view(n, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    return packed, (exp + 127).to(torch.uint8)


def pack_sf_atoms(sf: torch.Tensor) -> torch.Tensor:
    """``(N, K/32) u8`` → ``(ceil(N/128), ceil(K/128), 32, 4, 4)`` u8; padding scales are 2^0."""
    n, kb = sf.shape
    n_pad, kb_pad = -(-n // 128) * 128, -(-kb // 4) * 4
    full = torch.full((n_pad, kb_pad), 127, dtype=torch.uint8, device=sf.device)
    full[:n, :kb] = sf
    v = full.view(n_pad // 128, 4, 32, kb_pad // 4, 4)      # [nt, r//32, r%32, kt, kb]
    return v.permute(0, 3, 2, 1, 4).contiguous()             # [nt, kt, r%32, r//32, kb]


def unpack_sf_atoms(atoms: torch.Tensor, n: int, kb: int) -> torch.Tensor:
    nt, kt = atoms.shape[:2]
    v = atoms.permute(0, 3, 2, 1, 4).reshape(nt * 128, kt * 4)
    return v[:n, :kb].contiguous()


__all__ = [
    "GROUP", "quantize_e2m1", "quantize_mxfp4", "pack_sf_atoms", "unpack_sf_atoms",
    "dequant_mxfp4", "e8m0_to_float", "unpack_e2m1",
]
