"""Rank bookkeeping for tensor / data / expert parallelism.

One process drives one GPU. ``tp`` ranks share a model replica; ``dp`` replicas are
independent; with expert parallelism the experts of a MoE layer are sharded either over the
replicas (DP+EP) or over the tensor-parallel ranks of one replica (EP over TP). The
reference keeps the same facts in module globals (python/minisgl/distributed/info.py:18-98).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class RankInfo:
    rank: int
    size: int

    def __post_init__(self) -> None:
        if not (0 <= self.rank < self.size):
            raise ValueError(f"rank {self.rank} outside world of {self.size}")

    @property
    def is_primary(self) -> bool:
        return self.rank == 0


_TP: Optional[RankInfo] = None
_DP: Optional[RankInfo] = None
_EP_ENABLED: bool = False
_EP_OVER_TP: bool = False


def set_tp_info(rank: int, size: int) -> None:
    global _TP
    _TP = RankInfo(rank, size)


def set_dp_info(rank: int, size: int) -> None:
    global _DP
    _DP = RankInfo(rank, size)


def set_ep(enabled: bool, over_tp: bool = False) -> None:
    global _EP_ENABLED, _EP_OVER_TP
    _EP_ENABLED, _EP_OVER_TP = bool(enabled), bool(over_tp)


def reset_parallel_info() -> None:
    global _TP, _DP, _EP_ENABLED, _EP_OVER_TP
    _TP = _DP = None
    _EP_ENABLED = _EP_OVER_TP = False


def try_get_tp_info() -> Optional[RankInfo]:
    return _TP


def get_tp_info() -> RankInfo:
    return _TP if _TP is not None else RankInfo(0, 1)


def get_dp_info() -> RankInfo:
    return _DP if _DP is not None else RankInfo(0, 1)


def ep_enabled() -> bool:
    return _EP_ENABLED


def ep_over_tp() -> bool:
    return _EP_ENABLED and _EP_OVER_TP


def get_ep_info() -> RankInfo:
    """Rank and size of the group that shards experts."""
    if not _EP_ENABLED:
        return RankInfo(0, 1)
    return get_tp_info() if _EP_OVER_TP else get_dp_info()


def device_index(dp_rank: int, tp_rank: int, tp_size: int) -> int:
    """Replica-major placement: GPU = dp_rank * tp + tp_rank
    (python/minisgl/engine/config.py:266-276)."""
    return dp_rank * tp_size + tp_rank
