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
                 scheme=None, n_group: int = 1, topk_group: int = 1, selection_bias: bool = False,
                 gated: bool = True, act: str = "silu", expert_input: Optional[int] = None) -> None:
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
        # non-gated experts (down(act(up x)), Nemotron-H) take 16-bit weights and the local path only;
        # expert_input: width of the experts' input when a latent projection sits in front of them
        self._gated, self._act = gated, act
        self._in = expert_input or hidden
        self._n_group, self._topk_group = max(1, n_group), max(1, topk_group)
        self.gate = ReplicatedLinear(hidden, num_experts, dtype, device, None)
        if selection_bias:
            # DeepSeek-V3 / GLM-4 style: added to the scores when choosing experts, not to the weights
            self.e_score_correction_bias = torch.zeros((num_experts,), dtype=torch.float32, device=device)
        self.w13 = torch.empty((self._e_local, (2 if gated else 1) * self._i_local, self._in), dtype=dtype,
                               device=device)
        self.w2 = torch.empty((self._e_local, self._in, self._i_local), dtype=dtype, device=device)
        # Quantised experts keep their checkpoint precision on the GPU (the reference's expert
        # methods: python/minisgl/layers/moe.py:42-520):
        #   mxfp4        W4A8, e2m1 + UE8M0 scale atoms (re-encoding the stacks is lossless for an
        #                MXFP4 checkpoint, whose values are on that grid)
        #   fp8_block    W8A8 with 128 x 128 weight blocks and 1 x 128 activation groups; the loader
        #                hands over the checkpoint's own e4m3 values and scales (``_raw_fp8``)
        #   fp8_channel  W8A8 with one scale per (expert, output channel)
        name = str(getattr(scheme, "name", "")).lower() if scheme is not None else ""
        aligned = hidden % 128 == 0 and self._i_local % 128 == 0
        self._quant_kind = None
        if aligned and "mxfp4" in name:
            self._quant_kind = "mxfp4"
        elif aligned and name == "fp8_block" and tuple(getattr(scheme, "block", (128, 128))) == (128, 128):
            self._quant_kind = "fp8_block"
        elif aligned and name in ("fp8_channel", "fp8_tensor"):
            self._quant_kind = "fp8_channel"
        self._w4a8 = self._quant_kind == "mxfp4"
        self._raw_fp8 = None   # (w13_q, w13_scale, w2_q, w2_scale) straight from an fp8 checkpoint

    def forward(self, x: torch.Tensor, expert_x: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns this rank's partial result (tensor-parallel partial sum when the
        intermediate dimension is sharded; complete under expert parallelism). ``expert_x``: the
        experts' input when it differs from the router's (a latent projection in front of them)."""
        logits = self.gate.forward(x)
        if expert_x is not None:
            x = expert_x
        bias = getattr(self, "e_score_correction_bias", None)
        ctx = try_global_ctx()
        use_ep = self._ep is not None and ctx is not None and ctx.ep is not None
        counts = None
        if self._n_group > 1:
            from ..ops import ref

            topk_w, topk_ids = ref.moe_route_grouped(logits, self._k, self._renorm, self._scoring, bias,
                                                     self._routed_scale, self._n_group, self._topk_group)
        elif x.is_cuda and not use_ep and getattr(self, "_tier", None) is None:
            # the routing kernel also counts the tokens of every local expert for the alignment step
            from ..ops import cuda as K

            counts = torch.empty(self._e_local, dtype=torch.int32, device=x.device)
            topk_w, topk_ids = K.moe_route(logits, self._k, self._renorm, self._scoring, bias, self._routed_scale,
                                           counts, self._e_start, self._e_local)
        else:
            topk_w, topk_ids = ops.moe_route(logits, self._k, self._renorm, self._scoring, bias, self._routed_scale)
        if use_ep and self._gated:
            return ctx.ep.dispatch_compute_combine(self, x, topk_w, topk_ids)
        return self.local_experts(x, topk_w, topk_ids, counts)

    def local_experts(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor, counts=None
                      ) -> torch.Tensor:
        if not self._gated:
            return ops.moe_forward_plain(x, self.w13, self.w2, topk_w, topk_ids, self._e_start, counts, self._act)
        tier = getattr(self, "_tier", None)
        if tier is not None:
            return tier.forward(x, topk_w, topk_ids - self._e_start)
        packed = getattr(self, "_packed", None)
        if packed is not None:
            from ..ops.moe_kernels import moe_forward_quant

            return moe_forward_quant(self._quant_kind, x, packed, topk_w, topk_ids, self._e_start, counts)
        if self._act != "silu":
            # GELU-gated experts (Gemma-4): the grouped-GEMM kernels apply SiLU in their epilogue
            if x.is_cuda:
                raise NotImplementedError(f"no expert kernel with a {self._act} gate")
            from ..ops import ref

            return ref.moe_forward(x, self.w13, self.w2, topk_w, topk_ids, self._e_start, act=self._act)
        if x.is_cuda:
            from ..ops import cuda as K

            return K.moe_forward(x, self.w13, self.w2, topk_w, topk_ids, self._e_start, counts)
        return ops.moe_forward(x, self.w13, self.w2, topk_w, topk_ids, self._e_start)

    def expert_weights(self):
        """``(kind, tensors)`` of the resident expert stacks for the grouped-GEMM pipeline
        (``ops.moe_kernels.run_experts``)."""
        if getattr(self, "_tier", None) is not None:
            raise RuntimeError("experts paged in from the host tier have no resident stack")
        packed = getattr(self, "_packed", None)
        if packed is not None:
            return self._quant_kind, packed
        return "bf16", (self.w13, self.w2)

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

    def _encode_fp8(self) -> None:
        """fp8 expert stacks: the checkpoint's own tensors when the loader kept them, otherwise
        (random-init weights) a fresh quantisation of the 16-bit stacks."""
        dev = self.w13.device
        if self._raw_fp8 is not None:
            self._packed = tuple(t.to(dev).contiguous() for t in self._raw_fp8)
            self._raw_fp8 = None
        elif self._quant_kind == "fp8_block":
            def enc(w):  # [E, N, K] -> e4m3 [E, N, K], fp32 [E, N/128, K/128]
                e, n, k = w.shape
                qs, ss = [], []
                for i in range(e):
                    blocks = w[i].float().view(n // 128, 128, k // 128, 128)
                    scale = blocks.abs().amax((1, 3)).clamp_min(1e-8) / 448.0
                    qs.append((blocks / scale[:, None, :, None]).view(n, k).to(torch.float8_e4m3fn))
                    ss.append(scale)
                return torch.stack(qs).contiguous(), torch.stack(ss).float().contiguous()

            self._packed = enc(self.w13) + enc(self.w2)
        else:
            def enc(w):  # [E, N, K] -> e4m3 [E, N, K], fp32 [E, N]
                scale = w.float().abs().amax(-1).clamp_min(1e-8) / 448.0
                return (w.float() / scale[..., None]).to(torch.float8_e4m3fn).contiguous(), scale.float().contiguous()

            self._packed = enc(self.w13) + enc(self.w2)
        self.w13 = self.w13[:0]
        self.w2 = self.w2[:0]

    def _post_load_self(self) -> None:
        if self._w4a8 and self.w13.is_cuda and not type(self).offload_slots:
            self._encode_w4a8()
            return
        if self._quant_kind in ("fp8_block", "fp8_channel") and self.w13.is_cuda and not type(self).offload_slots:
            self._encode_fp8()
            return
        if self._raw_fp8 is not None:
            # CPU oracle path: expand the checkpoint tensors to the 16-bit stacks
            w13_q, w13_s, w2_q, w2_s = self._raw_fp8
            self._raw_fp8 = None

            def dense(q, s):
                if s.dim() == 3:
                    s = s.repeat_interleave(128, 1).repeat_interleave(128, 2)[:, : q.shape[1], : q.shape[2]]
                else:
                    s = s[..., None]
                return (q.float() * s.float()).to(self._compute_dtype)

            self.w13, self.w2 = dense(w13_q, w13_s), dense(w2_q, w2_s)
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
