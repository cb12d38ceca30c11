"""Paged pool of compressed attention latents (python/minisgl/kvcache/mla_pool.py:11-80).

A latent-attention layer can keep, per token, the normalised ``kv_lora_rank`` latent channels and
the one rotary key shared by all heads (``kv_lora_rank + qk_rope_head_dim`` values) instead of the
per-head keys and values expanded from them (``heads x (key width + value width)`` values): 576
against 10240 values per token and layer for GLM-4.7-Flash, 576 against 40960 for DeepSeek-V3.
Attention over this pool is the absorbed form (``ops.ref.mla_attention``): queries are moved into
the latent space with the key half of ``kv_b_proj``, the weighted latents come back through its
value half.

Layout ``[layers, pages + 1, page_size, width]``; page ``pages`` is the scratch page of padding rows.
"""
from __future__ import annotations

import torch

from .base import BaseKVCachePool


class MLALatentCache(BaseKVCachePool):
    latent = True
    fp8 = False

    def __init__(self, num_layers: int, num_pages: int, page_size: int, lora_rank: int, rope_dim: int, dtype,
                 device) -> None:
        self.num_layers, self.num_pages, self.page_size = num_layers, num_pages, page_size
        self.lora_rank, self.rope_dim = int(lora_rank), int(rope_dim)
        self.width = self.lora_rank + self.rope_dim
        self._buf = torch.zeros((num_layers, num_pages + 1, page_size, self.width), dtype=dtype, device=device)

    @property
    def dummy_page(self) -> int:
        return self.num_pages

    @property
    def device(self) -> torch.device:
        return self._buf.device

    @property
    def dtype(self) -> torch.dtype:
        return self._buf.dtype

    def rows(self, layer: int) -> torch.Tensor:
        """``[pages + 1, page_size, width]`` of one layer."""
        return self._buf[layer]

    def store(self, layer: int, latent: torch.Tensor, k_rot: torch.Tensor, out_loc: torch.Tensor) -> None:
        """``latent [T, lora]``, ``k_rot [T, rope]`` (rotary applied) to the token slots ``out_loc``."""
        flat = self._buf[layer].view(-1, self.width)
        flat.index_copy_(0, out_loc.long(), torch.cat([latent, k_rot], dim=-1).to(flat.dtype))

    # the interface of the multi-head cache ([pages, heads, page_size, dim]) with one "head" that is
    # key and value at once, for code that walks a pool without knowing its kind (state digests)
    def k_cache(self, layer: int) -> torch.Tensor:
        return self._buf[layer].unsqueeze(1)

    def v_cache(self, layer: int) -> torch.Tensor:
        return self._buf[layer].unsqueeze(1)

    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer: int) -> None:
        raise NotImplementedError("a latent pool takes store(layer, latent, k_rot, out_loc)")

    @staticmethod
    def token_bytes(num_layers: int, lora_rank: int, rope_dim: int, itemsize: int) -> int:
        return num_layers * (lora_rank + rope_dim) * itemsize
