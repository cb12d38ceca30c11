"""Parallel runtime: rank info, NCCL baseline communicator, symmetric peer memory and the
fused compute+collective kernels."""
from .info import (
    RankInfo,
    device_index,
    ep_enabled,
    ep_over_tp,
    get_dp_info,
    get_ep_info,
    get_tp_info,
    reset_parallel_info,
    set_dp_info,
    set_ep,
    set_tp_info,
    try_get_tp_info,
)

__all__ = [
    "RankInfo",
    "device_index",
    "ep_enabled",
    "ep_over_tp",
    "get_dp_info",
    "get_ep_info",
    "get_tp_info",
    "reset_parallel_info",
    "set_dp_info",
    "set_ep",
    "set_tp_info",
    "try_get_tp_info",
]
