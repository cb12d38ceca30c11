"""Host-RAM expert tier of one MoE layer.

All ``E`` experts stay in a pinned host arena; the device holds ``slots < E`` of them. Before the
expert MLPs run, the experts this step routes to are made resident: hits are touched in the SLRU
cache, misses are copied host→device with ``cudaMemcpyAsync`` on a side stream and the compute
stream waits on an event (python/minisgl/weights/moe_interpose.py:429, expert_cache.py:147;
the reference's slot indirection is ``set_expert_slot_map``). Routing ids are then rewritten from
expert ids to slot ids, so the grouped GEMM indexes the slab directly.

The choice of experts is made on the host, so a step that uses this tier runs eagerly (outside
CUDA graphs), as in the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .expert_cache import SLRUCache
from .pinned_arena import PinnedArena


class HostExpertTier:
    """``host_experts`` < E together with ``disk_dir`` adds a third tier: the pinned arena then holds
    only that many experts (its own SLRU cache) and every expert has a record in two flat files
    under ``disk_dir`` (weights/disk_tier.py); a device miss whose expert is not in the arena
    first reads the records into an arena slot, then uploads from there."""

    def __init__(self, w13: torch.Tensor, w2: torch.Tensor, slots: int, device, protected_fraction: float = 0.8,
                 host_experts: Optional[int] = None, disk_dir: Optional[str] = None, layer_index: int = 0) -> None:
        self.num_experts = w13.shape[0]
        self.slots = min(slots, self.num_experts)
        self.device = torch.device(device)
        self.arena = PinnedArena()
        self.disk = None
        self.host_cache: Optional[SLRUCache] = None
        if host_experts is not None and host_experts < self.num_experts:
            if not disk_dir:
                raise ValueError("a pinned arena smaller than the expert set needs a disk tier")
            if host_experts < self.slots:
                raise ValueError("the pinned arena must hold at least what the device slab holds")
            import os

            from .disk_tier import DiskExpertTier, ExpertFile

            os.makedirs(disk_dir, exist_ok=True)
            files = {}
            for name, w in (("w13", w13), ("w2", w2)):
                f = ExpertFile(os.path.join(disk_dir, f"layer{layer_index}.{name}.bin"), 1, self.num_experts,
                               tuple(w.shape[1:]), w.dtype)
                f.create()
                for e in range(self.num_experts):
                    f.write(0, e, w[e])
                files[name] = f
            self.disk = DiskExpertTier(files)
            self.host_cache = SLRUCache(host_experts, protected_fraction)
            rows = host_experts
        else:
            rows = self.num_experts
        # both families in one page-locked allocation (placement first, then a single pin)
        self.arena.reserve("w13", (rows,) + tuple(w13.shape[1:]), w13.dtype)
        self.arena.reserve("w2", (rows,) + tuple(w2.shape[1:]), w2.dtype)
        self.arena.attach()
        self.h13, self.h2 = self.arena.get("w13"), self.arena.get("w2")
        if self.disk is None:
            self.h13.copy_(w13)
            self.h2.copy_(w2)
        else:
            self.h13.zero_()
            self.h2.zero_()
        self.d13 = torch.empty((self.slots,) + tuple(w13.shape[1:]), dtype=w13.dtype, device=self.device)
        self.d2 = torch.empty((self.slots,) + tuple(w2.shape[1:]), dtype=w2.dtype, device=self.device)
        self.cache = SLRUCache(self.slots, protected_fraction)
        self.slot_map = torch.full((self.num_experts,), -1, dtype=torch.int32, device=self.device)
        self.copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.bytes_copied = 0
        # optional (RouteTrace, layer index): every step's routed experts are counted there
        self.trace = None
        self.layer_index = layer_index

    def _host_rows(self, experts: List[int]) -> Dict[int, int]:
        """Arena row of every expert in ``experts``, reading from disk what the arena lacks."""
        if self.host_cache is None:
            return {e: e for e in experts}
        rows: Dict[int, int] = {}
        missing: List[int] = []
        for e in experts:
            hit = self.host_cache.touch(e)
            if hit is None:
                missing.append(e)
            else:
                rows[e] = self.host_cache.slot_of(e)
        if missing:
            if self.copy_stream is not None:
                # an arena row may still be the source of an upload queued earlier
                self.copy_stream.synchronize()
            for e in missing:
                slot, _ = self.host_cache.admit(e, pinned=experts)
                rows[e] = slot
            self.disk.fetch(0, missing, {"w13": [self.h13[rows[e]] for e in missing],
                                         "w2": [self.h2[rows[e]] for e in missing]})
        return rows

    def prewarm(self, experts: List[int]) -> None:
        """Make the hottest experts of an earlier run's route trace resident before the first step
        (python/minisgl/weights/route_trace.py: hot sets seed the cache at boot)."""
        self.ensure_resident(list(experts)[: self.slots])

    def ensure_resident(self, expert_ids: List[int]) -> None:
        need = sorted(set(int(e) for e in expert_ids if 0 <= int(e) < self.num_experts))
        if len(need) > self.slots:
            raise RuntimeError(f"step routes to {len(need)} experts but the device slab holds {self.slots}")
        misses = [e for e in need if self.cache.touch(e) is None]
        if not misses:
            return
        updates: Dict[int, int] = {}
        evicted: List[int] = []
        for e in misses:
            slot, old = self.cache.admit(e, pinned=need)
            updates[e] = slot
            if old is not None:
                evicted.append(old)
        rows = self._host_rows(list(updates.keys()))
        if self.copy_stream is not None:
            # the slab may still be read by kernels queued earlier on the compute stream
            self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.copy_stream):
                for e, slot in updates.items():
                    self.d13[slot].copy_(self.h13[rows[e]], non_blocking=True)
                    self.d2[slot].copy_(self.h2[rows[e]], non_blocking=True)
            torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)
        else:
            for e, slot in updates.items():
                self.d13[slot].copy_(self.h13[rows[e]])
                self.d2[slot].copy_(self.h2[rows[e]])
        per_expert = self.h13[0].numel() * self.h13.element_size() + self.h2[0].numel() * self.h2.element_size()
        self.bytes_copied += per_expert * len(updates)
        idx = torch.tensor(list(updates.keys()) + evicted, dtype=torch.int64)
        val = torch.tensor(list(updates.values()) + [-1] * len(evicted), dtype=torch.int32)
        self.slot_map[idx.to(self.device)] = val.to(self.device)

    def _run(self, x, topk_w, topk_ids) -> torch.Tensor:
        from .. import ops

        slot_ids = self.slot_map[topk_ids.long().clamp(0, self.num_experts - 1)]
        valid = (topk_ids >= 0) & (topk_ids < self.num_experts)
        slot_ids = torch.where(valid, slot_ids, torch.full_like(slot_ids, -1))
        return ops.moe_forward(x, self.d13, self.d2, topk_w, slot_ids.to(torch.int32), 0)

    def forward(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        """A step that routes to more experts than the slab holds (a wide prefill) runs in rounds:
        each round makes one slab-full of experts resident and adds their contribution (the
        reference stages such prefills through a separate slab, weights/prefill_stage.py:116)."""
        routed = topk_ids.reshape(-1).tolist()
        if self.trace is not None:
            self.trace.record(self.layer_index, routed)
        need = sorted(set(int(e) for e in routed if 0 <= int(e) < self.num_experts))
        if len(need) <= self.slots:
            self.ensure_resident(need)
            return self._run(x, topk_w, topk_ids)
        out = None
        for i in range(0, len(need), self.slots):
            chunk = need[i:i + self.slots]
            self.ensure_resident(chunk)
            member = torch.zeros(self.num_experts + 1, dtype=torch.bool, device=topk_ids.device)
            member[torch.tensor(chunk, device=topk_ids.device)] = True
            ids = torch.where(member[topk_ids.long().clamp(-1, self.num_experts - 1)], topk_ids,
                              torch.full_like(topk_ids, -1))
            part = self._run(x, topk_w, ids).float()
            out = part if out is None else out + part
        return out.to(x.dtype)
