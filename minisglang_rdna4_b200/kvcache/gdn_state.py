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
        self._arena = None                      # pinned frames for snapshots kept on the host
        self.stream = None                      # the stream the snapshot / restore copies are issued on
        self._frames: Dict[object, int] = {}    # snapshot key -> frame

    def attach_host_arena(self, budget_bytes: int) -> int:
        """Keep snapshots in page-locked host frames (one slab, ``budget_bytes`` of it) instead of
        device memory; returns the number of frames (python/minisgl/kvcache/host_arena.py:132)."""
        from .host_arena import FrameLayout, PinnedFrameArena

        layout = FrameLayout([("conv", tuple(self.conv[:, 0].shape), self.conv.dtype),
                              ("ssm", tuple(self.ssm[:, 0].shape), torch.float32)])
        frames = layout.frames_in(budget_bytes)
        if frames <= 0:
            return 0
        self._arena = PinnedFrameArena(layout, frames, pin=self.conv.is_cuda)
        return frames

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

    def snapshot(self, slot: int, key, host: bool = True, end: int = 0) -> None:
        if self._arena is not None:
            frame = self._arena.alloc()
            if frame is not None:
                v = self._arena.views(frame)
                v["conv"].copy_(self.conv[:, slot], non_blocking=True)
                v["ssm"].copy_(self.ssm[:, slot], non_blocking=True)
                self._frames[key] = frame
                self._snapshots[key] = (v["conv"], v["ssm"])
                return
            # every frame is held: this snapshot stays on the device
        conv, ssm = self.conv[:, slot].clone(), self.ssm[:, slot].clone()
        if host and conv.is_cuda and self._arena is None:
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
        frame = self._frames.pop(key, None)
        if frame is not None:
            ev = None
            if self.conv.is_cuda:
                # a restore from this frame (or the copy that filled it) may still be queued
                ev = torch.cuda.Event()
                ev.record(self.stream) if self.stream is not None else ev.record()
            self._arena.release(frame, ev)

    @property
    def num_snapshots(self) -> int:
        return len(self._snapshots)
