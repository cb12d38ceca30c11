"""The paged-attention backend: one implementation for prefill, chunked extend over a cached
prefix, decode, and speculative verification (plain or with a tree mask). All of them read K
and V from the paged pool after the fused norm/RoPE/store kernel has written this step's
rows, so a cached prefix needs no special path. The reference keeps several backends
(python/minisgl/attention/__init__.py:19-98); on sm_100a one suffices.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..core import Batch, get_global_ctx
from .base import AttnMetadata, BaseAttnBackend


class PagedAttentionBackend(BaseAttnBackend):
    def __init__(self, num_q_heads: int, num_kv_heads: int, head_dim: int, device,
                 max_batch: int = 0, max_seq_len: int = 0, single_split: bool = False) -> None:
        self.hq, self.hk, self.d = num_q_heads, num_kv_heads, head_dim
        self.device = device
        # The number of KV splits of a decode step depends only on the batch size and the
        # longest sequence the pool can hold, never on the lengths in the batch: a captured
        # graph and an eager step then reduce in the same order and agree bit for bit.
        # ``single_split`` pins it to one (speculative verification must reproduce decode).
        self.max_seq_len = max_seq_len
        self.single_split = single_split
        self._workspace: Optional[torch.Tensor] = None
        if torch.device(device).type == "cuda":
            from ..ops import cuda as K

            self._workspace = K.attention_workspace(max(max_batch, 1), num_q_heads, head_dim, device)
            K.force_general_decode_attention(single_split)

    def prepare_metadata(self, batch: Batch, block_table, cu_q, seq_lens, max_q: int, max_kv: int,
                         causal: bool = True, mask: Optional[torch.Tensor] = None,
                         host_cu_q=None, host_seq_lens=None, mask_window: int = 0, mask_swa=None) -> None:
        """``host_cu_q`` / ``host_seq_lens`` are the same lengths as numpy arrays: a prefill-phase
        step on a GPU builds the tables of the tensor-core prefill kernel from them (every such
        step whose KV rows number at most 16 times its query rows: every prefill and chunked-prefill
        step whatever its size, so that a row's result does not depend on how its prompt was chunked;
        a short extend over a long cached prefix reads the pool in place with the general kernel).
        Decode and verification steps stay on the general kernel."""
        plan = None
        if (host_cu_q is not None and batch.is_prefill and not batch.spec_verify and mask is None and causal
                and self._workspace is not None and self.d == 128 and (self.hq // self.hk) % 2 == 0):
            from ..env import ENV
            from ..ops import cuda as K

            if not ENV.DISABLE_TC_PREFILL.value:
                b = int(len(host_seq_lens))
                t_pad = int(((host_seq_lens.astype("int64") + 127) // 128 * 128).sum()) if b else 0
                if K.tc_prefill_pays(int(host_cu_q[b]), t_pad):
                    plan = K.PrefillPlan(host_cu_q, host_seq_lens, self.device)
        batch.attn_metadata = AttnMetadata(
            cu_q=cu_q, seq_lens=seq_lens, block_table=block_table, max_q=max_q, max_kv=max_kv,
            decode=(max_q == 1 and plan is None), causal=causal, mask=mask, mask_window=mask_window, mask_swa=mask_swa,
            workspace=self._workspace,
            prefill_plan=plan,
        )

    def forward(self, q, layer: int, batch: Batch, *, scale: float, window: int = 0, swa: bool = False):
        md = batch.attn_metadata
        ctx = get_global_ctx()
        # a sliding-window layer with a pool of its own reads that pool through the step's second block table
        pool = ctx.swa_kv_cache if swa else ctx.kv_cache
        block_table = batch.swa_block_table if swa else md.block_table
        fp8 = getattr(pool, "fp8", False)
        if md.prefill_plan is not None and not window:
            from ..ops import cuda as K

            k_cache = pool.k_cache(layer)
            if K.prefill_attention_tc_ok(q, k_cache, causal=md.causal, window=window, mask=md.mask, decode=False):
                return K.prefill_attention_tc(
                    q, k_cache, pool.v_cache(layer), block_table, md.prefill_plan, scale,
                    k_scale=pool.k_scale[layer] if fp8 else None, v_scale=pool.v_scale[layer] if fp8 else None)
        splits = 1
        if md.decode and not self.single_split and q.is_cuda:
            from ..ops.cuda import choose_splits

            splits = choose_splits(md.seq_lens.numel(), self.hk, self.max_seq_len or md.max_kv, True)
        mask = md.mask_swa if (window and md.mask_swa is not None) else md.mask
        return ops.paged_attention(
            q, pool.k_cache(layer), pool.v_cache(layer), block_table, md.cu_q, md.seq_lens, scale,
            causal=md.causal, window=window, mask=mask, mask_window=md.mask_window,
            k_scale=pool.k_scale[layer] if fp8 else None,
            v_scale=pool.v_scale[layer] if fp8 else None,
            max_q=md.max_q, max_kv=md.max_kv, decode=md.decode, workspace=md.workspace, splits=splits,
        )
