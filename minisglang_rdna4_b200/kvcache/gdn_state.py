"""Per-request recurrent state of the gated-delta-net layers.

Every linear-attention layer keeps, per request slot (the request's row of the page table), the
last ``kernel - 1`` inputs of its causal convolution and one ``[Dk, Dv]`` fp32 state matrix per
value head. Unlike K/V pages this state is a running summary: it cannot be rewound or shared
between requests, so a prefix-cache hit is only usable when a snapshot of the state at exactly
the matched length exists (``snapshot`` / ``restore``; python/minisgl/kvcache/gdn_state.py:45-372,
python/minisgl/scheduler/recurrent_slots.py:48-94).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch


class GDNStateCache:
    def __init__(self, num_layers: int, num_slots: int, conv_dim: int, conv_kernel: int, num_v_heads: int,
                 head_k_dim: int, head_v_dim: int, dtype: torch.dtype, device) -> None:
        self.num_layers, self.num_slots = num_layers, num_slots
        self.conv = torch.zeros((num_layers, num_slots, conv_dim, conv_kernel - 1), dtype=dtype, device=device)
        self.ssm = torch.zeros((num_layers, num_slots, num_v_heads, head_k_dim, head_v_dim), dtype=torch.float32,
                               device=device)
        self._snapshots: Dict[object, Tuple[torch.Tensor, torch.Tensor]] = {}

    @staticmethod
    def slot_bytes(num_layers: int, conv_dim: int, conv_kernel: int, num_v_heads: int, dk: int, dv: int,
                   itemsize: int) -> int:
        return num_layers * (conv_dim * (conv_kernel - 1) * itemsize + num_v_heads * dk * dv * 4)

    def conv_state(self, layer: int) -> torch.Tensor:
        return self.conv[layer]

    def ssm_state(self, layer: int) -> torch.Tensor:
        return self.ssm[layer]

    # ---- speculative verify: keep the state of a batch's slots and put (some of) them back ----
    def save_slots(self, slots: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Copies of the states of ``slots`` over all layers (``[L, B, ...]``), taken before a verify
        forward advances them by rows that may be rejected (python/minisgl/gdn/layer.py:640-760,
        the rollback half of verify-replay)."""
        idx = slots.long()
        return self.conv.index_select(1, idx), self.ssm.index_select(1, idx)

    def load_slots(self, slots: torch.Tensor, saved: Tuple[torch.Tensor, torch.Tensor],
                   which: Optional[torch.Tensor] = None) -> None:
        """Puts saved states back; ``which`` selects entries of the saved batch."""
        idx = slots.long()
        conv, ssm = saved
        if which is not None:
            w = which.long()
            conv, ssm, idx = conv.index_select(1, w), ssm.index_select(1, w), idx.index_select(0, w)
        self.conv.index_copy_(1, idx, conv)
        self.ssm.index_copy_(1, idx, ssm)

    # ---- snapshots: the state of one slot after exactly ``key`` tokens ----
    def slot_nbytes(self) -> int:
        """Bytes of one request's state over all recurrent layers (= the size of a snapshot)."""
        return int(self.conv[:, 0].numel() * self.conv.element_size() + self.ssm[:, 0].numel() * 4)

    def snapshot(self, slot: int, key, host: bool = True) -> None:
        conv, ssm = self.conv[:, slot].clone(), self.ssm[:, slot].clone()
        if host and conv.is_cuda:
            conv, ssm = conv.to("cpu", non_blocking=True), ssm.to("cpu", non_blocking=True)
        self._snapshots[key] = (conv, ssm)

    def restore(self, slot: int, key) -> bool:
        snap = self._snapshots.get(key)
        if snap is None:
            return False
        self.conv[:, slot].copy_(snap[0], non_blocking=True)
        self.ssm[:, slot].copy_(snap[1], non_blocking=True)
        return True

    def drop_snapshot(self, key) -> None:
        self._snapshots.pop(key, None)

    @property
    def num_snapshots(self) -> int:
        return len(self._snapshots)
