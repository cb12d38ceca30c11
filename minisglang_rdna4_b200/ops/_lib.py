"""ctypes binding of ``libmsgl_cuda.so`` (built in-tree by ``minisglang_rdna4_b200.build``).

The library exports plain C entry points that take raw device pointers and a stream handle;
there is no dependency on the PyTorch C++ ABI. On a machine with a GPU a missing library is
an error: the CUDA path never falls back to eager PyTorch silently.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmsgl_cuda.so")
# built with -DMSGL_CHECK_BOUNDS (python -m minisglang_rdna4_b200.build --checked); chosen by MSGL_CHECK_BOUNDS=1
CHECKED_LIB_PATH = os.path.join(_HERE, "libmsgl_cuda_checked.so")


def _wanted_lib() -> str:
    flag = (os.environ.get("MSGL_CHECK_BOUNDS") or os.environ.get("MINISGL_CHECK_BOUNDS") or "").strip().lower()
    if flag in ("1", "true", "yes", "on") and os.path.exists(CHECKED_LIB_PATH):
        return CHECKED_LIB_PATH
    return LIB_PATH

c_p = ctypes.c_void_p
c_i = ctypes.c_int
c_ll = ctypes.c_longlong
c_f = ctypes.c_float

_SIGNATURES = {
    "msgl_last_error": (ctypes.c_char_p, []),
    "msgl_embedding": (c_i, [c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p]),
    "msgl_rms_norm": (c_i, [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_f, c_i, c_i, c_p]),
    "msgl_act_and_mul": (c_i, [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p]),
    "msgl_quant_fp8": (c_i, [c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p]),
    "msgl_qk_norm_rope_store": (c_i, [c_p] * 11 + [c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_i, c_i, c_i, c_i, c_i, c_p]),
    "msgl_store_kv": (c_i, [c_p] * 7 + [c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p]),
    "msgl_gemm": (c_i, [c_i, c_p, c_ll, c_p, c_p, c_ll, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_i, c_i, c_i, c_p]),
    "msgl_gemm_tp": (c_i, [c_i, c_p, c_ll, c_p, c_p, c_ll, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_i, c_p, c_p]),
    "msgl_gemm_splitk_plan": (c_i, [c_i, c_i, c_i]),
    "msgl_gemm_splitk": (c_i, [c_i, c_p, c_ll, c_p, c_p, c_ll, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_i, c_i, c_p, c_p,
                               c_p]),
    "msgl_gemm_splitk_planes": (c_i, [c_i, c_p, c_ll, c_p, c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_i, c_p]),
    "msgl_rms_norm_planes": (c_i, [c_p, c_i, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_f, c_i, c_i, c_p]),
    "msgl_gemm_status": (c_i, [c_i]),
    "msgl_gemm_pair_mode": (c_i, [c_i]),
    "msgl_gemm_static_weights": (c_i, [c_i]),
    "msgl_set_pdl": (c_i, [c_i]),
    "msgl_attn_make_kv_map": (c_i, [c_p, c_p, c_i, c_i, c_i, c_i, c_ll, c_i]),
    "msgl_attn_workspace_floats": (c_ll, [c_i, c_i, c_i, c_i]),
    "msgl_paged_attention": (c_i, [c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_p, c_p, c_ll, c_p,
                                   c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_i,
                                   c_f, c_i, c_p]),
    "msgl_attn_status": (c_i, [c_i]),
    "msgl_attn_prefill_tc": (c_i, [c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_ll, c_i, c_p, c_i, c_p, c_p, c_p, c_i,
                                   c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_f, c_i, c_p]),
    "msgl_attn_tc_status": (c_i, [c_i]),
    "msgl_attn_force_general_decode": (None, [c_i]),
    "msgl_attn_decode_stages": (None, [c_i]),
    "msgl_argmax": (c_i, [c_p, c_p, c_i, c_i, c_ll, c_p]),
    "msgl_sample": (c_i, [c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_p]),
}

_lib: Optional[ctypes.CDLL] = None


class NativeLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _wanted_lib()
        if not os.path.exists(path):
            raise NativeLibraryMissing(
                f"{path} is missing: run `python -m minisglang_rdna4_b200.build` "
                "(the CUDA ops have no eager fallback)")
        handle = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def bind(name: str, restype, argtypes) -> None:
    """Register the signature of an entry point added by another module (comm, moe …)."""
    _SIGNATURES[name] = (restype, argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype, fn.argtypes = restype, argtypes


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().msgl_last_error()
        kinds = {1: "bad argument", 2: "CUDA error", 3: "device wait timed out"}
        raise RuntimeError(f"{what}: {kinds.get(rc, rc)}: {msg.decode() if msg else ''}")
