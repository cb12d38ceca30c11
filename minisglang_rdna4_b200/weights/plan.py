"""Placement plan of the expert weights over the memory tiers
(python/minisgl/weights/plan.py:1614, placement.py:756-786, host_capacity.py).

Given the expert geometry of a model and the budgets of each tier the resolver answers, per MoE
layer: how many experts get a device slot, how many stay in pinned host memory, how many are left
to the disk tier. Every rank computes the plan from the same inputs; ``digest`` is what the ranks
compare before loading (the reference exchanges it with ``all_gather_object``,
weights/plan.py:1427) so that a mismatch is reported at boot instead of as diverging routing.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional


@dataclass(frozen=True)
class ExpertGeometry:
    num_moe_layers: int
    num_experts: int          # per layer, on this rank (after expert parallelism)
    experts_per_token: int
    bytes_per_expert: int     # gate/up + down of one expert in the storage dtype


@dataclass(frozen=True)
class TierBudgets:
    device_bytes: int                    # for expert slots, all MoE layers together
    host_bytes: Optional[int] = None     # pinned; None = whatever the host check allows
    disk: bool = False                   # a disk tier exists for what the host cannot hold


@dataclass
class LayerPlacement:
    device_slots: int
    host_experts: int
    disk_experts: int


@dataclass
class OffloadPlan:
    geometry: ExpertGeometry
    layers: List[LayerPlacement] = field(default_factory=list)
    notes: List[str] = field(default_factory=list)

    @property
    def offloaded(self) -> bool:
        return any(p.device_slots < self.geometry.num_experts for p in self.layers)

    @property
    def device_bytes(self) -> int:
        return sum(p.device_slots for p in self.layers) * self.geometry.bytes_per_expert

    @property
    def host_bytes(self) -> int:
        return sum(p.host_experts for p in self.layers) * self.geometry.bytes_per_expert

    def to_dict(self) -> Dict:
        return {"geometry": asdict(self.geometry), "layers": [asdict(p) for p in self.layers]}

    @property
    def digest(self) -> str:
        return hashlib.sha256(json.dumps(self.to_dict(), sort_keys=True).encode()).hexdigest()[:16]


class PlanError(ValueError):
    pass


def min_device_slots(geo: ExpertGeometry, max_step_tokens: int = 1) -> int:
    """A decode step of ``t`` tokens routes to at most ``t * k`` distinct experts; the slab must
    hold one step's experts (wider prefills run in slab-sized rounds). Two steps' worth keeps the
    experts of the step in flight resident while the next step's misses are copied in."""
    need = min(geo.num_experts, max(1, max_step_tokens) * geo.experts_per_token)
    return min(geo.num_experts, max(2 * geo.experts_per_token, need))


def resolve_plan(geo: ExpertGeometry, budgets: TierBudgets, max_step_tokens: int = 1) -> OffloadPlan:
    """Uniform slots per layer (every layer is visited once per token, so no layer deserves more
    than another without a route trace); whole experts only."""
    plan = OffloadPlan(geo)
    if geo.num_moe_layers <= 0 or geo.num_experts <= 0:
        return plan
    per_layer = budgets.device_bytes // max(geo.bytes_per_expert * geo.num_moe_layers, 1)
    floor = min_device_slots(geo, max_step_tokens)
    slots = min(geo.num_experts, max(int(per_layer), floor))
    if per_layer < floor:
        plan.notes.append(f"device budget holds {int(per_layer)} experts per layer; raised to the minimum of {floor}")
    rest = geo.num_experts - slots
    # the host tier keeps a copy of EVERY expert that is not pinned to the device for good:
    # with fewer slots than experts any expert can be evicted, so all of them need a host home
    host_need = geo.num_experts if rest > 0 else 0
    host_cap = host_need
    if budgets.host_bytes is not None:
        host_cap = min(host_need, budgets.host_bytes // max(geo.bytes_per_expert * geo.num_moe_layers, 1))
    disk = host_need - host_cap
    if disk > 0 and not budgets.disk:
        raise PlanError(
            f"{host_need} experts per layer need a host copy but the pinned budget holds {host_cap} and there is "
            "no disk tier")
    if disk > 0 and host_cap < slots:
        raise PlanError("the pinned host tier must at least hold what the device slab can hold")
    plan.layers = [LayerPlacement(slots, int(host_cap), int(disk)) for _ in range(geo.num_moe_layers)]
    return plan


def check_agreement(digests: List[str]) -> None:
    """Raise when the ranks resolved different plans (first differing rank in the message)."""
    for rank, d in enumerate(digests):
        if d != digests[0]:
            raise PlanError(f"offload plan of rank {rank} ({d}) differs from rank 0 ({digests[0]})")
