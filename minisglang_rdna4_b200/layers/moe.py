"""Mixture-of-experts layer: router → top-k → grouped expert MLP → weighted combine, with
tensor-parallel (intermediate dimension sharded) and expert-parallel (whole experts sharded)
placements (python/minisgl/layers/moe.py:1008-1446).

Expert weights are stacked: ``w13 [E_local, 2I, H]`` (gate rows then up rows) and
``w2 [E_local, H, I]``. Under expert parallelism every rank runs the router on its own
tokens; ``parallel/ep.py`` moves token rows to the ranks that own the selected experts and
brings the weighted results back.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..core import try_global_ctx
from ..parallel.info import ep_enabled, get_ep_info, get_tp_info
from ..utils import div_even
from .base import BaseOP
from .linear import ReplicatedLinear


class MoELayer(BaseOP):
    # experts kept on the device per layer when the host-RAM expert tier is on (0 = all resident);
    # set by the engine from --expert-cache-gb before the weights are post-processed
    offload_slots: int = 0
    # pinned host rows per layer (0 = all experts) and the directory of the disk tier behind them
    offload_host_experts: int = 0
    offload_disk_dir: str = ""
    _tier_seq: int = 0

    def __init__(self, hidden: int, inter: int, num_experts: int, top_k: int, renormalize: bool,
                 dtype, device, scoring: str = "softmax", routed_scale: float = 1.0,
                 scheme=None) -> None:
        tp = get_tp_info()
        ep = get_ep_info()
        self._ep = ep if ep_enabled() else None
        self._E, self._k = num_experts, top_k
        self._renorm, self._scoring, self._routed_scale = renormalize, scoring, routed_scale
        if self._ep is not None:
            self._e_local = div_even(num_experts, self._ep.size)
            self._e_start = self._ep.rank * self._e_local
            self._i_local = inter
        else:
            self._e_local, self._e_start = num_experts, 0
            self._i_local = div_even(inter, tp.size)
        self._hidden = hidden
        self._compute_dtype = dtype
        self.gate = ReplicatedLinear(hidden, num_experts, dtype, device, None)
        self.w13 = torch.empty((self._e_local, 2 * self._i_local, hidden), dtype=dtype, device=device)
        self.w2 = torch.empty((self._e_local, hidden, self._i_local), dtype=dtype, device=device)
        # MXFP4 experts run W4A8 on the GPU: the stacks are (re-)encoded to e2m1 + UE8M0 scale
        # atoms after loading (lossless for an MXFP4 checkpoint, whose values are on that grid)
        self._w4a8 = scheme is not None and "mxfp4" in str(getattr(scheme, "name", "")).lower() \
            and hidden % 128 == 0 and self._i_local % 128 == 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Returns this rank's partial result (tensor-parallel partial sum when the
        intermediate dimension is sharded; complete under expert parallelism)."""
        logits = self.gate.forward(x)
        topk_w, topk_ids = ops.moe_route(logits, self._k, self._renorm, self._scoring, None,
                                         self._routed_scale)
        ctx = try_global_ctx()
        if self._ep is not None and ctx is not None and ctx.ep is not None:
            return ctx.ep.dispatch_compute_combine(self, x, topk_w, topk_ids)
        return self.local_experts(x, topk_w, topk_ids)

    def local_experts(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        tier = getattr(self, "_tier", None)
        if tier is not None:
            return tier.forward(x, topk_w, topk_ids - self._e_start)
        packed = getattr(self, "_packed", None)
        if packed is not None:
            from ..ops.moe_kernels import moe_forward_w4a8

            return moe_forward_w4a8(x, *packed, topk_w, topk_ids, self._e_start)
        return ops.moe_forward(x, self.w13, self.w2, topk_w, topk_ids, self._e_start)

    def _encode_w4a8(self) -> None:
        from ..quant import mxfp4

        def enc(w):  # [E, N, K] 16-bit → packed [E, N, K/2], atoms [E, N/128, K/128, 32, 4, 4]
            e, n, k = w.shape
            packed, sf = mxfp4.quantize_mxfp4(w.reshape(e * n, k))
            atoms = torch.stack([mxfp4.pack_sf_atoms(sf[i * n:(i + 1) * n]) for i in range(e)])
            return packed.view(e, n, k // 2).contiguous(), atoms.contiguous()

        p13, a13 = enc(self.w13)
        p2, a2 = enc(self.w2)
        self._packed = (p13, a13, p2, a2)
        self.w13 = self.w13[:0]
        self.w2 = self.w2[:0]

    def _post_load_self(self) -> None:
        if self._w4a8 and self.w13.is_cuda and not type(self).offload_slots:
            self._encode_w4a8()
            return
        slots = type(self).offload_slots
        if slots and slots < self._e_local:
            from ..weights import HostExpertTier

            cls = type(self)
            host = cls.offload_host_experts if 0 < cls.offload_host_experts < self._e_local else None
            self._tier = HostExpertTier(self.w13, self.w2, slots, self.w13.device, host_experts=host,
                                        disk_dir=cls.offload_disk_dir or None, layer_index=cls._tier_seq)
            cls._tier_seq += 1
            # the full stacks now live in pinned host memory only
            self.w13 = self.w13[:0]
            self.w2 = self.w2[:0]

    @property
    def needs_tp_reduce(self) -> bool:
        """True when ``forward`` returns a partial sum over the tensor-parallel group: the
        intermediate dimension is sharded, or whole experts are sharded over the TP ranks (every
        rank sees every token, computes its own experts, and the sum over ranks completes it;
        python/minisgl/layers/moe.py:1258-1269)."""
        from ..parallel.info import ep_over_tp

        if get_tp_info().size == 1:
            return False
        return self._ep is None or ep_over_tp()

    def init_dummy(self, gen: torch.Generator, std: float = 0.02) -> None:
        for name in ("w13", "w2"):
            t = getattr(self, name)
            w = torch.randn(t.shape, generator=gen, device=gen.device, dtype=torch.float32) * std
            setattr(self, name, w.to(t.device, t.dtype))
        self.gate.init_dummy(gen, std)
