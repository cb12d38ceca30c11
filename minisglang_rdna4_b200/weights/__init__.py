"""Expert weight tiers for models whose experts do not fit in device memory
(python/minisgl/weights/): a pinned host arena that holds every expert, a device slab with room
for a subset, and an SLRU residency cache that decides which experts stay on the device. Misses
are filled with ``cudaMemcpyAsync`` on a side stream. Around them: the placement plan resolver
(``plan``), a device-memory ledger (``accounting``), the pinned-memory capacity check
(``host_capacity``), the routing trace that seeds the cache (``route_trace``), a disk tier for what
the host cannot hold (``disk_tier``) and the boot timeline (``boot_timeline``)."""
from .accounting import MemoryLedger
from .boot_timeline import BootTimeline
from .disk_tier import DiskExpertTier, ExpertFile
from .expert_cache import SLRUCache
from .host_tier import HostExpertTier
from .pinned_arena import PinnedArena
from .plan import ExpertGeometry, OffloadPlan, PlanError, TierBudgets, resolve_plan
from .route_trace import RouteTrace

__all__ = ["SLRUCache", "HostExpertTier", "PinnedArena", "MemoryLedger", "BootTimeline", "DiskExpertTier",
           "ExpertFile", "ExpertGeometry", "OffloadPlan", "PlanError", "TierBudgets", "resolve_plan", "RouteTrace"]
