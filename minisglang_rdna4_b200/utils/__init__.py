"""Small shared helpers: logging, integer arithmetic, registries, NVTX ranges."""
from .logger import init_logger
from .misc import (
    Registry,
    align_ceil,
    align_down,
    call_if_main,
    cdiv,
    div_even,
    next_pow2,
    nvtx_range,
    nvtx_annotate,
    UNSET,
    Unset,
)

__all__ = [
    "init_logger",
    "Registry",
    "align_ceil",
    "align_down",
    "call_if_main",
    "cdiv",
    "div_even",
    "next_pow2",
    "nvtx_range",
    "nvtx_annotate",
    "UNSET",
    "Unset",
]
