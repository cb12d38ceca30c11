"""Expert weight tiers for models whose experts do not fit in device memory
(python/minisgl/weights/): a pinned host arena that holds every expert, a device slab with room
for a subset, and an SLRU residency cache that decides which experts stay on the device. Misses
are filled with ``cudaMemcpyAsync`` on a side stream."""
from .expert_cache import SLRUCache
from .host_tier import HostExpertTier
from .pinned_arena import PinnedArena

__all__ = ["SLRUCache", "HostExpertTier", "PinnedArena"]
