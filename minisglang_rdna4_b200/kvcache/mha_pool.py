"""Paged multi-head KV pool.

Layout ``[2, layers, pages, kv_heads, page_size, head_dim]`` (head-major inside a page) so
that one (page, head) tile is a contiguous ``page_size x head_dim`` block: the decode and
extend attention kernels fetch it with one bulk copy. With ``fp8`` storage the pool holds
e4m3 bytes and a float32 descale per (layer, kv head) for K and for V
(``value = byte * descale``; python/minisgl/kvcache/mha_pool.py:37-43,55-270 keeps the same
per-head scales). Page ``num_pages`` (one past the end) is a scratch page for padded
requests of a captured graph.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import BaseKVCachePool


class MHAKVCache(BaseKVCachePool):
    def __init__(
        self,
        num_layers: int,
        num_pages: int,
        page_size: int,
        num_kv_heads: int,
        head_dim: int,
        dtype: torch.dtype,
        device: torch.device,
        fp8: bool = False,
        geometry=None,
    ) -> None:
        # geometry: (kv heads, head width) per layer for models whose layers differ (Gemma-4: wide global
        # heads, narrower sliding ones). Every layer then gets rows of the widest layer's size and views the
        # front of each page as its own [heads, page_size, width] block. 16-bit, tensor-op paths only: the
        # views are strided and the kernels take dense pools.
        self._views = None
        if geometry is not None and len(set(geometry)) > 1:
            if fp8:
                raise ValueError("a pool with per-layer head geometry is 16-bit only")
            if len(geometry) != num_layers:
                raise ValueError("one (heads, width) pair per layer")
            self.geometry = [(int(h), int(d)) for h, d in geometry]
            num_kv_heads, head_dim = 1, max(h * d for h, d in self.geometry)
        elif geometry is not None:
            num_kv_heads, head_dim = geometry[0]
        self.num_layers = num_layers
        self.num_pages = num_pages
        self.page_size = page_size
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.compute_dtype = dtype
        self.fp8 = fp8
        store_dtype = torch.float8_e4m3fn if fp8 else dtype
        # +1: the dummy page written by padded rows of a graph replay
        self._buf = torch.zeros(
            (2, num_layers, num_pages + 1, num_kv_heads, page_size, head_dim),
            dtype=store_dtype,
            device=device,
        )
        self.k_scale = torch.ones((num_layers, num_kv_heads), dtype=torch.float32, device=device)
        self.v_scale = torch.ones((num_layers, num_kv_heads), dtype=torch.float32, device=device)
        # calibration run (16-bit pool only): running |max| per (layer, head) of every row written
        self.amax: Optional[torch.Tensor] = None
        if getattr(self, "geometry", None) is not None:
            pages, ps, width = num_pages + 1, page_size, head_dim
            self._views = [[self._buf[which, layer].view(pages, ps * width)[:, : h * ps * d].view(pages, h, ps, d)
                            for layer, (h, d) in enumerate(self.geometry)] for which in (0, 1)]

    # ---- calibration of the fp8 descales (python/minisgl/kvcache/mha_pool.py:123-270) ----
    def start_calibration(self) -> None:
        """Record the largest |value| per (layer, kv head) of all K / V rows stored from now on.
        Runs against a 16-bit pool, so the first calibration of a model does not need fp8 scales."""
        if self.fp8:
            raise ValueError("calibrate the fp8 KV scales on a 16-bit pool (--kv-dtype auto)")
        self.amax = torch.zeros((2, self.num_layers, self.num_kv_heads), dtype=torch.float32, device=self.device)

    def observe_written(self, layer: int, out_loc: torch.Tensor) -> None:
        """Fold the rows just stored at token slots ``out_loc`` of ``layer`` into the running amax."""
        if self.amax is None or out_loc.numel() == 0:
            return
        loc = out_loc.long()
        page, off = loc // self.page_size, loc % self.page_size
        keep = page < self.num_pages                       # padded graph rows write the dummy page
        page, off = page[keep], off[keep]
        for which in (0, 1):
            rows = self._buf[which, layer][page, :, off]   # [n, heads, dim]
            if rows.numel():
                self.amax[which, layer] = torch.maximum(self.amax[which, layer], rows.float().abs().amax(dim=(0, 2)))

    def finish_calibration(self, margin: float = 1.0):
        """Descales ``(k_scale, v_scale)`` ``[layers, heads]`` = amax * margin / 448; a head that saw
        no data keeps 1.0. Ends the recording."""
        from .fp8_scales import FP8_MAX

        if self.amax is None:
            raise ValueError("no calibration is running")
        amax, self.amax = self.amax, None
        scales = torch.where(amax > 0, amax * margin / FP8_MAX, torch.ones_like(amax)).clamp_min(1e-6)
        return scales[0].cpu(), scales[1].cpu()

    # ---- accessors ----
    @property
    def dummy_page(self) -> int:
        return self.num_pages

    def k_cache(self, layer: int) -> torch.Tensor:
        return self._buf[0, layer] if self._views is None else self._views[0][layer]

    def v_cache(self, layer: int) -> torch.Tensor:
        return self._buf[1, layer] if self._views is None else self._views[1][layer]

    @property
    def device(self) -> torch.device:
        return self._buf.device

    @property
    def dtype(self) -> torch.dtype:
        return self._buf.dtype

    @property
    def bytes_per_token(self) -> int:
        return 2 * self.num_layers * self.num_kv_heads * self.head_dim * self._buf.element_size()

    @staticmethod
    def token_bytes(num_layers: int, kv_heads: int, head_dim: int, itemsize: int) -> int:
        return 2 * num_layers * kv_heads * head_dim * itemsize

    def set_scales(self, k_scale: torch.Tensor, v_scale: torch.Tensor) -> None:
        """Install per-(layer, head) descales (amax / 448)."""
        self.k_scale.copy_(k_scale.to(self.k_scale))
        self.v_scale.copy_(v_scale.to(self.v_scale))

    # ---- writes ----
    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer: int) -> None:
        """Scatter ``k``/``v`` rows ``[T, kv_heads, head_dim]`` to token slots ``out_loc``."""
        from ..ops import store_kv

        store_kv(
            k, v, self.k_cache(layer), self.v_cache(layer), out_loc,
            self.k_scale[layer] if self.fp8 else None,
            self.v_scale[layer] if self.fp8 else None,
        )

    # ---- reads (reference path and tests) ----
    def gather(self, layer: int, slots: torch.Tensor, which: int) -> torch.Tensor:
        """Rows ``[len(slots), kv_heads, head_dim]`` in compute precision."""
        page = slots // self.page_size
        off = slots % self.page_size
        rows = self._buf[which, layer][page, :, off]  # [n, heads, dim]
        if self.fp8:
            scale = (self.k_scale if which == 0 else self.v_scale)[layer]
            return rows.to(torch.float32) * scale[None, :, None]
        return rows
