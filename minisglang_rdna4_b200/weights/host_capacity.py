"""Can this host pin what the plan wants to pin? (python/minisgl/weights/host_capacity.py).
Page-locking more than the machine can spare fails late and badly (the allocator stalls or the
OOM killer picks a victim), so the check runs before the first ``pin_memory`` call."""
from __future__ import annotations

import resource
from typing import Callable, Optional, Tuple


def _meminfo_available(read: Optional[Callable[[], str]] = None) -> Optional[int]:
    try:
        text = read() if read is not None else open("/proc/meminfo").read()
    except OSError:
        return None
    for line in text.splitlines():
        if line.startswith("MemAvailable:"):
            return int(line.split()[1]) * 1024
    return None


def pinned_budget(reserve_fraction: float = 0.2, read_meminfo: Optional[Callable[[], str]] = None,
                  memlock: Optional[Tuple[int, int]] = None) -> Optional[int]:
    """Bytes that may be page-locked: available memory minus a reserve for the page cache and the
    process itself, capped by RLIMIT_MEMLOCK when that limit is finite (CUDA's pinned allocations
    are not charged to it on Linux, but container runtimes that set it usually mean it)."""
    avail = _meminfo_available(read_meminfo)
    if avail is None:
        return None
    budget = int(avail * (1.0 - reserve_fraction))
    soft = (memlock if memlock is not None else resource.getrlimit(resource.RLIMIT_MEMLOCK))[0]
    if soft not in (resource.RLIM_INFINITY, -1) and soft > (1 << 30):
        budget = min(budget, int(soft))
    return budget


def check_pinned(nbytes: int, **kw) -> None:
    budget = pinned_budget(**kw)
    if budget is not None and nbytes > budget:
        raise MemoryError(
            f"the offload plan wants {nbytes / (1 << 30):.1f} GiB of pinned host memory; this host can spare "
            f"{budget / (1 << 30):.1f} GiB")
