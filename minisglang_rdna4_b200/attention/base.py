"""Attention backend interface (python/minisgl/attention/base.py:18)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Optional

import torch

from ..core import Batch


@dataclass
class AttnMetadata:
    cu_q: torch.Tensor          # [B+1] int32 prefix sums of query lengths
    seq_lens: torch.Tensor      # [B] int32 KV length including the tokens of this step
    block_table: torch.Tensor   # [B, P] int32 page ids
    max_q: int
    max_kv: int
    decode: bool                # every request has exactly one query row
    causal: bool = True
    mask: Optional[torch.Tensor] = None   # additive [T, >= max_kv] bias for tree verification
    mask_window: int = 0                  # > 0: mask rows [T, mask_window] cover the last mask_window KV positions only
    mask_swa: Optional[torch.Tensor] = None   # the mask sliding-window layers take instead (a mask replaces the window rule)
    workspace: Optional[torch.Tensor] = None
    prefill_plan: Optional[object] = None  # ops.cuda.PrefillPlan of a prefill-phase step on a GPU


class BaseAttnBackend(ABC):
    @abstractmethod
    def prepare_metadata(self, batch: Batch, block_table: torch.Tensor, cu_q: torch.Tensor,
                         seq_lens: torch.Tensor, max_q: int, max_kv: int) -> None: ...

    @abstractmethod
    def forward(self, q: torch.Tensor, layer: int, batch: Batch, *, scale: float, window: int = 0
                ) -> torch.Tensor: ...
