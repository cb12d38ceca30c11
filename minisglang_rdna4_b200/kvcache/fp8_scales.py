"""Per-(layer, kv-head) descales of the fp8 KV cache: where they come from and how they are
calibrated (python/minisgl/kvcache/fp8_scales.py:37-38,203-340).

Resolution order: a side-car ``kv_scales*.safetensors`` next to the checkpoint (tensors
``k_scale`` / ``v_scale`` of shape ``[layers, kv_heads]`` = amax / 448, full head count, sharded
here by tensor-parallel rank) → per-layer ``…self_attn.k_scale`` / ``v_scale`` tensors in the
checkpoint → identity (1.0). ``KVScaleCalibrator`` records running amax values from bf16 K/V
rows during a calibration run and writes such a side-car.
"""
from __future__ import annotations

import glob
import os
import re
from typing import Dict, Optional, Tuple

import torch

FP8_MAX = 448.0


def find_sidecar(model_path: str, tp_size: int = 1) -> Optional[str]:
    if not model_path or not os.path.isdir(model_path):
        return None
    exact = os.path.join(model_path, f"kv_scales_tp{tp_size}.safetensors")
    if os.path.exists(exact):
        return exact
    hits = sorted(glob.glob(os.path.join(model_path, "kv_scales*.safetensors")))
    return hits[0] if hits else None


def _shard_heads(t: torch.Tensor, tp_rank: int, tp_size: int, total_heads: int) -> torch.Tensor:
    if tp_size == 1 or t.shape[1] != total_heads:
        return t
    if total_heads >= tp_size:
        per = total_heads // tp_size
        return t[:, tp_rank * per:(tp_rank + 1) * per]
    group = tp_size // total_heads
    return t[:, tp_rank // group: tp_rank // group + 1]


def resolve_kv_scales(model_path: str, num_layers: int, kv_heads_total: int, tp_rank: int = 0, tp_size: int = 1,
                      checkpoint_tensors: Optional[Dict[str, torch.Tensor]] = None
                      ) -> Tuple[torch.Tensor, torch.Tensor, str]:
    """Returns ``(k_scale, v_scale, source)`` with shape ``[layers, local kv heads]``."""
    local = max(kv_heads_total // tp_size, 1)
    side = find_sidecar(model_path, tp_size)
    if side is not None:
        from safetensors.torch import load_file

        d = load_file(side)
        k, v = d["k_scale"].float(), d["v_scale"].float()
        if k.shape[0] != num_layers:
            raise ValueError(f"{side}: {k.shape[0]} layers, model has {num_layers}")
        return (_shard_heads(k, tp_rank, tp_size, kv_heads_total).contiguous(),
                _shard_heads(v, tp_rank, tp_size, kv_heads_total).contiguous(), f"sidecar:{os.path.basename(side)}")
    if checkpoint_tensors:
        k = torch.ones(num_layers, local)
        v = torch.ones(num_layers, local)
        found = 0
        for name, t in checkpoint_tensors.items():
            m = re.match(r"model\.layers\.(\d+)\.self_attn\.(?:attn\.)?([kv])_scale$", name)
            if not m:
                continue
            layer, which = int(m.group(1)), m.group(2)
            if layer >= num_layers:
                continue
            (k if which == "k" else v)[layer] = t.float().reshape(-1)[:1].expand(local) if t.numel() == 1 \
                else _shard_heads(t.float().reshape(1, -1), tp_rank, tp_size, kv_heads_total)[0]
            found += 1
        if found:
            return k, v, "checkpoint"
    return torch.ones(num_layers, local), torch.ones(num_layers, local), "identity"


class KVScaleCalibrator:
    """Running amax per (layer, kv head) of the K and V rows seen in a calibration run."""

    def __init__(self, num_layers: int, kv_heads: int) -> None:
        self.k_amax = torch.zeros(num_layers, kv_heads)
        self.v_amax = torch.zeros(num_layers, kv_heads)

    def observe(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """``k`` / ``v`` ``[tokens, kv_heads, head_dim]`` (after norm and RoPE)."""
        self.k_amax[layer] = torch.maximum(self.k_amax[layer], k.float().abs().amax(dim=(0, 2)).cpu())
        self.v_amax[layer] = torch.maximum(self.v_amax[layer], v.float().abs().amax(dim=(0, 2)).cpu())

    def scales(self, margin: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
        k = (self.k_amax * margin / FP8_MAX).clamp_min(1e-6)
        v = (self.v_amax * margin / FP8_MAX).clamp_min(1e-6)
        return k, v

    def save(self, path: str, margin: float = 1.0) -> None:
        from safetensors.torch import save_file

        k, v = self.scales(margin)
        save_file({"k_scale": k.contiguous(), "v_scale": v.contiguous()}, path)
