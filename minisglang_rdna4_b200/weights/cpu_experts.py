"""CPU expert tier: experts whose 4-bit weights stay in host memory are evaluated by the host
library (``csrc/host/cpu_moe.cpp``) instead of being copied to the GPU for a few tokens.

The reference ships this as ``libcpumoe.so`` with a ctypes front end
(tools/cpu_moe/cpu_moe_so.cpp:316-476, python/minisgl/weights/moe_interpose.py:429). Here the
tier is a small class: ``set_expert`` registers e2m1 codes + per-group scales of one expert,
``forward`` runs the routed SwiGLU MLPs for a batch of tokens and returns the gate-weighted
sum. ``reference`` is the fp32 PyTorch restatement the tests compare against.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import numpy as np
import torch

from ..ops.host import host_lib

E2M1 = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32)


def _bind(lib) -> None:
    if getattr(lib, "_cpumoe_bound", False):
        return
    c = ctypes
    lib.msgl_cpumoe_create.restype = c.c_void_p
    lib.msgl_cpumoe_create.argtypes = [c.c_int] * 5
    lib.msgl_cpumoe_destroy.restype = None
    lib.msgl_cpumoe_destroy.argtypes = [c.c_void_p]
    lib.msgl_cpumoe_set_expert.restype = c.c_int
    lib.msgl_cpumoe_set_expert.argtypes = [c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p]
    lib.msgl_cpumoe_isa.restype = c.c_int
    lib.msgl_cpumoe_isa.argtypes = [c.c_void_p, c.c_int]
    lib.msgl_cpumoe_forward.restype = c.c_int
    lib.msgl_cpumoe_forward.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                                        c.c_int]
    lib._cpumoe_bound = True


def dequant_e2m1(codes: torch.Tensor, scales: torch.Tensor, group: int) -> torch.Tensor:
    """``codes (N, K/2) u8`` (low nibble = even element) and ``scales (N, K/group) f32`` → fp32 ``(N, K)``."""
    lo = (codes & 15).long()
    hi = (codes >> 4).long()
    vals = torch.stack([E2M1[lo], E2M1[hi]], dim=-1).reshape(codes.shape[0], -1)
    return vals * scales.repeat_interleave(group, dim=1)


class CpuExpertTier:
    def __init__(self, num_experts: int, hidden: int, inter: int, group: int = 32, threads: int = 0) -> None:
        lib = host_lib()
        if lib is None or not hasattr(lib, "msgl_cpumoe_create"):
            raise RuntimeError("libmsgl_host.so is missing the CPU expert tier; run python -m minisglang_rdna4_b200.build")
        _bind(lib)
        self._lib = lib
        self.num_experts, self.hidden, self.inter, self.group = num_experts, hidden, inter, group
        self._h = lib.msgl_cpumoe_create(num_experts, hidden, inter, group, threads)
        if not self._h:
            raise ValueError("unsupported CPU expert tier shape (group must be 16 or 32 and divide both dims)")
        self._keep: Dict[int, Tuple[torch.Tensor, ...]] = {}

    def close(self) -> None:
        if self._h:
            self._lib.msgl_cpumoe_destroy(self._h)
            self._h = None

    def __del__(self) -> None:  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass

    @property
    def isa(self) -> str:
        return ("scalar", "avx512-fp32", "avx512-vnni-int8")[self._lib.msgl_cpumoe_isa(self._h, 1)]

    def set_expert(self, e: int, w13: torch.Tensor, s13: torch.Tensor, w2: torch.Tensor, s2: torch.Tensor) -> None:
        """``w13 (2*inter, hidden/2) u8`` gate rows then up rows, ``s13 (2*inter, hidden/group) f32``,
        ``w2 (hidden, inter/2) u8``, ``s2 (hidden, inter/group) f32``. The tier keeps references
        (pinned host tensors in the engine), it does not copy."""
        tensors = tuple(t.contiguous() for t in (w13, s13.float(), w2, s2.float()))
        assert tensors[0].shape == (2 * self.inter, self.hidden // 2) and tensors[0].dtype == torch.uint8
        assert tensors[2].shape == (self.hidden, self.inter // 2) and tensors[2].dtype == torch.uint8
        assert tensors[1].shape == (2 * self.inter, self.hidden // self.group)
        assert tensors[3].shape == (self.hidden, self.inter // self.group)
        self._keep[e] = tensors
        rc = self._lib.msgl_cpumoe_set_expert(self._h, e, *[t.data_ptr() for t in tensors])
        if rc:
            raise IndexError(f"expert {e} out of range")

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                int8_activations: bool = False) -> torch.Tensor:
        """``x (T, hidden)``, ``topk_ids (T, k) int`` (negative = skip), ``topk_weights (T, k)`` →
        ``(T, hidden)`` fp32 on the CPU."""
        xf = x.detach().to("cpu", torch.float32).contiguous()
        ids = topk_ids.detach().to("cpu", torch.int32).contiguous()
        w = topk_weights.detach().to("cpu", torch.float32).contiguous()
        out = torch.empty_like(xf)
        rc = self._lib.msgl_cpumoe_forward(self._h, xf.data_ptr(), ids.data_ptr(), w.data_ptr(), out.data_ptr(),
                                           xf.shape[0], ids.shape[1], int(int8_activations))
        if rc:
            raise RuntimeError("cpu expert tier forward failed")
        return out

    def reference(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        xf = x.detach().to("cpu", torch.float32)
        out = torch.zeros_like(xf)
        for t in range(xf.shape[0]):
            for j in range(topk_ids.shape[1]):
                e = int(topk_ids[t, j])
                if e < 0 or e not in self._keep:
                    continue
                w13, s13, w2, s2 = self._keep[e]
                w13f = dequant_e2m1(w13, s13, self.group)
                w2f = dequant_e2m1(w2, s2, self.group)
                gu = w13f @ xf[t]
                act = torch.nn.functional.silu(gu[: self.inter]) * gu[self.inter:]
                out[t] += float(topk_weights[t, j]) * (w2f @ act)
        return out
