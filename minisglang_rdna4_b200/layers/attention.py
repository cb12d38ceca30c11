"""Attention layer: fused QK-norm + RoPE + KV store, then paged attention through the
backend in the global context (python/minisgl/layers/attention.py:19-141)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..core import get_global_ctx
from ..models.config import RotaryConfig
from .base import BaseOP
from .rotary import get_rope_cache


class AttentionLayer(BaseOP):
    _non_persistent = ("_cos_sin",)

    def __init__(self, layer_id: int, num_q_local: int, num_kv_local: int, head_dim: int,
                 rotary: RotaryConfig, eps: float, dtype, device,
                 window: int = 0, scale: Optional[float] = None) -> None:
        self._layer_id = layer_id
        self._hq, self._hk, self._d = num_q_local, num_kv_local, head_dim
        self._rotary = rotary
        self._eps = eps
        self._window = window
        self._scale = scale if scale is not None else head_dim ** -0.5
        self._device = device
        self._cos_sin: Optional[torch.Tensor] = None
        # which pool holds this layer's K/V and at which layer index: the engine re-numbers the layers
        # when sliding-window layers get a pool of their own
        self._swa = False
        self._kv_index = layer_id
        # a layer that reads the K/V another layer stored (same positions, same pool rows) and stores nothing:
        # the other layer's decoder index; the engine resolves it to that layer's pool and row
        self._kv_donor: Optional[int] = None

    def forward(self, qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor] = None,
                k_norm_w: Optional[torch.Tensor] = None) -> torch.Tensor:
        ctx = get_global_ctx()
        batch = ctx.batch
        if self._cos_sin is None:
            self._cos_sin = get_rope_cache(self._rotary, qkv.device)
        pool = ctx.swa_kv_cache if self._swa else ctx.kv_cache
        layer = self._kv_index
        out_loc = batch.swa_out_loc if self._swa else batch.out_loc
        if self._kv_donor is not None:          # qkv holds the queries only
            q = ops.q_norm_rope(qkv, q_norm_w, batch.positions, self._cos_sin, self._hq, self._d,
                                self._rotary.rotary_dim, self._eps, self._rotary.interleaved)
            out = ctx.attn_backend.forward(q, layer, batch, scale=self._scale, window=self._window, swa=self._swa)
            return out.reshape(out.shape[0], self._hq * self._d)
        k_scale = pool.k_scale[layer] if pool.fp8 else None
        v_scale = pool.v_scale[layer] if pool.fp8 else None
        q = ops.qk_norm_rope_store(
            qkv, q_norm_w, k_norm_w,
            batch.positions, self._cos_sin, self._hq, self._hk, self._d, self._rotary.rotary_dim,
            self._eps, pool.k_cache(layer), pool.v_cache(layer), out_loc, k_scale, v_scale,
            self._rotary.interleaved,
        )
        if getattr(pool, "amax", None) is not None:
            pool.observe_written(layer, out_loc)
        out = ctx.attn_backend.forward(q, layer, batch, scale=self._scale, window=self._window, swa=self._swa)
        return out.reshape(out.shape[0], self._hq * self._d)
