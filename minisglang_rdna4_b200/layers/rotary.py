"""Rotary-embedding tables, shared between layers with identical parameters
(python/minisgl/layers/rotary.py:13-262)."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..models.config import RotaryConfig
from ..ops.ref import build_cos_sin_cache

_CACHE: Dict[Tuple, torch.Tensor] = {}


def get_rope_cache(cfg: RotaryConfig, device) -> torch.Tensor:
    """``[max_position, rotary_dim]`` float32 table (cos ‖ sin) on ``device``."""
    key = cfg.key() + (str(device),)
    table = _CACHE.get(key)
    if table is None:
        table = build_cos_sin_cache(cfg.rotary_dim, cfg.max_position, cfg.base, cfg.scaling).to(device)
        _CACHE[key] = table
    return table


def clear_rope_cache() -> None:
    _CACHE.clear()
