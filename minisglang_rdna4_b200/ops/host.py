"""Host-side native helpers (C++), loaded with ctypes.

``libmsgl_host.so`` is built from ``csrc/host/*.cpp``: the radix-tree key comparison
(the reference has the same helper in python/minisgl/kernel/csrc/src/radix.cpp:19-40), the
page free-list and the CPU expert GEMV. Each function has a NumPy restatement that is used
when the library has not been built and that the unit tests compare against.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmsgl_host.so")
_lib: Optional[ctypes.CDLL] = None
_tried = False


def host_lib() -> Optional[ctypes.CDLL]:
    global _lib, _tried
    if _tried:
        return _lib
    _tried = True
    if os.path.exists(_LIB_PATH):
        lib = ctypes.CDLL(_LIB_PATH)
        lib.msgl_common_prefix_i32.restype = ctypes.c_int64
        lib.msgl_common_prefix_i32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        _lib = lib
    return _lib


def common_prefix_len_numpy(a: np.ndarray, b: np.ndarray, limit: int) -> int:
    n = min(limit, len(a), len(b))
    if n == 0:
        return 0
    diff = np.flatnonzero(a[:n] != b[:n])
    return int(diff[0]) if diff.size else n


def common_prefix_len(a: np.ndarray, b: np.ndarray, limit: int) -> int:
    """Length of the common prefix of two int32 arrays, capped at ``limit``."""
    lib = host_lib()
    n = min(limit, len(a), len(b))
    if lib is None or n < 64:
        return common_prefix_len_numpy(a, b, n)
    a = np.ascontiguousarray(a[:n])
    b = np.ascontiguousarray(b[:n])
    return int(lib.msgl_common_prefix_i32(a.ctypes.data, b.ctypes.data, n))
