"""Linear methods: which tensors a (possibly quantised) linear layer owns, how they are
repacked after loading, and which kernel multiplies with them.

Execution modes on sm_100a:

===============  =========================  ==========================================
scheme           weights in HBM             tensor-core path
===============  =========================  ==========================================
none             bf16 ``(N, K)``            ``kind::f16``
fp8_channel      e4m3 + ``(N,)`` f32        ``kind::f8f6f4``; per-token × per-channel
                                            scales applied in the epilogue (W8A8)
fp8_tensor       as fp8_channel (scale broadcast)
fp8_block        e4m3 + 128x128 f32 scales  ``kind::f8f6f4``: every 128-deep K block accumulates in
                                            its own tensor-memory buffer and is promoted with
                                            (1 x 128 activation scale) x (block scale) by the
                                            epilogue warps (``csrc/gemm_fp8_block.cu``); other
                                            block shapes are expanded to 16-bit at load
mxfp4            packed e2m1 + UE8M0/32     ``kind::mxf8f6f4.block_scale`` against e4m3
                                            activations (W4A8); per-token scale in epilogue
nvfp4, int4      see ``NvFp4Method`` / ``Int4Method``
===============  =========================  ==========================================

The reference's method table is python/minisgl/quant/method.py:352-949.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple, Union

import torch

from .. import ops
from . import int4 as int4_codec
from . import mxfp4 as mx_codec
from . import nvfp4 as nv_codec
from .config import (
    SCHEME_FP8_BLOCK, SCHEME_FP8_CHANNEL, SCHEME_FP8_TENSOR, SCHEME_INT4, SCHEME_MXFP4,
    SCHEME_NONE, SCHEME_NVFP4, QuantScheme,
)


@dataclass
class ActQ:
    """A per-token e4m3 activation: ``x ≈ q * scale[:, None]``. Produced by a fused
    norm/activation kernel so that the consuming GEMM does not re-read bf16."""

    q: torch.Tensor
    scale: torch.Tensor
    # set when peers are still delivering the rows (parallel.symm.ReadyRows): the consuming
    # GEMM waits per 128-row block; any other consumer calls get_comm().wait_ready first
    ready: object = None

    @property
    def shape(self):
        return self.q.shape


LinearInput = Union[torch.Tensor, ActQ]


class LinearMethod:
    """Strategy object attached to a linear layer."""

    wants_act_quant = False   # True when ``apply`` prefers an ``ActQ`` input

    def create_weights(self, n: int, k: int, dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def shard_dims(self) -> Dict[str, Tuple[int, int]]:
        """Per tensor name: (dim that follows the output dim N, dim that follows K), or -1."""
        raise NotImplementedError

    def process_after_load(self, layer) -> None:
        return None

    def apply(self, layer, x: LinearInput, bias: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def init_dummy(self, layer, gen: torch.Generator, std: float = 0.02) -> None:
        """Fill the layer with N(0, std) weights expressed in this scheme."""
        raise NotImplementedError


def _dequant_input(x: LinearInput, dtype: torch.dtype) -> torch.Tensor:
    if isinstance(x, ActQ):
        return (x.q.float() * x.scale.float()[:, None]).to(dtype)
    return x


def _randn(shape, gen: torch.Generator, std: float, device) -> torch.Tensor:
    # generate on the generator's device in chunks to bound peak memory
    return torch.randn(shape, generator=gen, device=gen.device, dtype=torch.float32).mul_(std).to(device)


class UnquantizedMethod(LinearMethod):
    def create_weights(self, n, k, dtype, device):
        return {"weight": torch.empty((n, k), dtype=dtype, device=device)}

    def shard_dims(self):
        return {"weight": (0, 1)}

    def apply(self, layer, x, bias):
        return ops.gemm(_dequant_input(x, layer.weight.dtype), layer.weight, bias)

    def init_dummy(self, layer, gen, std=0.02):
        layer.weight = _randn(layer.weight.shape, gen, std, layer.weight.device).to(layer.weight.dtype)


class Fp8ChannelMethod(LinearMethod):
    """W8A8: e4m3 weights with one scale per output channel, dynamic per-token activations
    (python/minisgl/quant/method.py:923-939)."""

    wants_act_quant = True

    def __init__(self, per_tensor: bool = False) -> None:
        self.per_tensor = per_tensor

    def create_weights(self, n, k, dtype, device):
        return {
            "weight": torch.empty((n, k), dtype=torch.float8_e4m3fn, device=device),
            "weight_scale": torch.empty((n, 1), dtype=torch.float32, device=device),
        }

    def shard_dims(self):
        return {"weight": (0, 1), "weight_scale": (0, -1)}

    def process_after_load(self, layer):
        layer.weight_scale = layer.weight_scale.float().reshape(-1).contiguous()
        layer._out_dtype = layer._compute_dtype

    def apply(self, layer, x, bias):
        if not isinstance(x, ActQ):
            x = ActQ(*ops.per_token_quant_fp8(x))
        return ops.gemm_w8a8(x.q, x.scale, layer.weight, layer.weight_scale, layer._compute_dtype, bias)

    def init_dummy(self, layer, gen, std=0.02):
        n, k = layer.weight.shape
        w = _randn((n, k), gen, std, layer.weight.device)
        scale = w.abs().amax(-1, keepdim=True).clamp_min(1e-8) / 448.0
        layer.weight = (w / scale).to(torch.float8_e4m3fn)
        layer.weight_scale = scale.float()


class Fp8BlockMethod(LinearMethod):
    """e4m3 weights with 128x128 scale blocks, activations quantised in 1x128 groups
    (python/minisgl/quant/method.py:846-897)."""

    def __init__(self, block: Tuple[int, int] = (128, 128)) -> None:
        self.block = block

    def create_weights(self, n, k, dtype, device):
        bn, bk = self.block
        return {
            "weight": torch.empty((n, k), dtype=torch.float8_e4m3fn, device=device),
            "weight_scale_inv": torch.empty((-(-n // bn), -(-k // bk)), dtype=torch.float32, device=device),
        }

    def shard_dims(self):
        return {"weight": (0, 1), "weight_scale_inv": (0, 1)}

    def process_after_load(self, layer):
        layer.weight_scale_inv = layer.weight_scale_inv.float().contiguous()
        n, k = layer.weight.shape
        if self.block != (128, 128) or k % 128 != 0:
            # odd block shapes are expanded to 16-bit once
            ws = layer.weight_scale_inv.repeat_interleave(self.block[0], 0).repeat_interleave(self.block[1], 1)
            layer._dense = (layer.weight.float() * ws[:n, :k]).to(layer._compute_dtype)

    def apply(self, layer, x, bias):
        dense = getattr(layer, "_dense", None)
        if dense is not None:
            return ops.gemm(_dequant_input(x, dense.dtype), dense, bias)
        xin = _dequant_input(x, layer._compute_dtype)
        xq, xs = ops.per_group_quant_fp8(xin, 128)
        y = ops.gemm_fp8_block(xq, xs, layer.weight, layer.weight_scale_inv, layer._compute_dtype)
        return y if bias is None else y + bias

    def init_dummy(self, layer, gen, std=0.02):
        n, k = layer.weight.shape
        bn, bk = self.block
        w = _randn((n, k), gen, std, layer.weight.device)
        npad, kpad = -(-n // bn) * bn, -(-k // bk) * bk
        wp = torch.zeros((npad, kpad), device=w.device)
        wp[:n, :k] = w
        blocks = wp.view(npad // bn, bn, kpad // bk, bk)
        scale = blocks.abs().amax((1, 3)).clamp_min(1e-8) / 448.0
        q = (blocks / scale[:, None, :, None]).view(npad, kpad)[:n, :k]
        layer.weight = q.to(torch.float8_e4m3fn).contiguous()
        layer.weight_scale_inv = scale.float()


class MxFp4Method(LinearMethod):
    """W4A8: packed e2m1 weights + UE8M0 scale per 32, per-token e4m3 activations
    (python/minisgl/quant/method.py:589-598)."""

    wants_act_quant = True

    def create_weights(self, n, k, dtype, device):
        return {
            "weight_packed": torch.empty((n, k // 2), dtype=torch.uint8, device=device),
            "weight_scale": torch.empty((n, k // 32), dtype=torch.uint8, device=device),
        }

    def shard_dims(self):
        return {"weight_packed": (0, 1), "weight_scale": (0, 1)}

    def process_after_load(self, layer):
        layer._n, layer._k = layer.weight_packed.shape[0], layer.weight_packed.shape[1] * 2
        if layer.weight_packed.is_cuda:
            layer._sf_atoms = mx_codec.pack_sf_atoms(layer.weight_scale)
            # the 4-bit tensor map wants K in whole 128-element blocks (a row-parallel shard of an
            # odd intermediate size is not): pad the rows with zero codes; the activation's K block
            # past its end is filled with zeros by TMA, so the padding contributes nothing
            k_pad = (layer._k + 127) // 128 * 128
            if k_pad != layer._k:
                layer.weight_packed = torch.nn.functional.pad(layer.weight_packed, (0, (k_pad - layer._k) // 2))

    def apply(self, layer, x, bias):
        if not isinstance(x, ActQ):
            x = ActQ(*ops.per_token_quant_fp8(x))
        return ops.gemm_w4a8_mxfp4(
            x.q, x.scale, layer.weight_packed, layer.weight_scale,
            getattr(layer, "_sf_atoms", None), layer._compute_dtype, bias,
        )

    def init_dummy(self, layer, gen, std=0.02):
        n, k2 = layer.weight_packed.shape
        dev = layer.weight_packed.device
        rows = max(1, (1 << 24) // (k2 * 2))
        packed, scales = [], []
        for r0 in range(0, n, rows):
            w = _randn((min(rows, n - r0), k2 * 2), gen, std, dev)
            p, s = mx_codec.quantize_mxfp4(w)
            packed.append(p)
            scales.append(s)
        layer.weight_packed = torch.cat(packed)
        layer.weight_scale = torch.cat(scales)


def _w4_native_ok(n: int, k: int, group: int, device) -> bool:
    """Shapes the 4-bit-resident GEMM takes (``csrc/gemm_w4a16.cu``); anything else is expanded."""
    return torch.device(device).type == "cuda" and n % 8 == 0 and k % 64 == 0 and \
        (group == 16 or (group >= 32 and group % 32 == 0)) and k % group == 0


class NvFp4Method(LinearMethod):
    """NVFP4 checkpoint tensors (e2m1 codes, an e4m3 scale per 16 elements, a per-channel factor;
    python/minisgl/quant/method.py:729-749). On the GPU the codes stay 4-bit in HBM and are expanded
    inside the GEMM (W4A16: 16-bit activations, weights exact); on the CPU oracle path, and for
    shapes the kernel does not take, they are expanded once after loading."""

    def __init__(self, divides: bool) -> None:
        self.divides = divides

    def create_weights(self, n, k, dtype, device):
        return {
            "weight_packed": torch.empty((n, k // 2), dtype=torch.uint8, device=device),
            "weight_scale": torch.empty((n, k // 16), dtype=torch.float8_e4m3fn, device=device),
            "weight_global_scale": torch.empty((n,), dtype=torch.float32, device=device),
        }

    def shard_dims(self):
        return {"weight_packed": (0, 1), "weight_scale": (0, 1), "weight_global_scale": (0, -1)}

    def process_after_load(self, layer):
        n, k = layer.weight_packed.shape[0], layer.weight_packed.shape[1] * 2
        if _w4_native_ok(n, k, 16, layer.weight_packed.device) and layer._compute_dtype in (torch.bfloat16, torch.float16):
            layer._w4 = (layer.weight_packed.contiguous(),
                         layer.weight_scale.view(torch.uint8).t().contiguous(),       # [K/16, N] e4m3 bytes
                         layer.weight_global_scale.float().contiguous())
            layer.weight_scale = layer.weight_scale[:0]
            return
        layer._dense = nv_codec.dequant_nvfp4(
            layer.weight_packed, layer.weight_scale, layer.weight_global_scale
        ).to(layer._compute_dtype)
        layer.weight_packed = layer.weight_packed[:0]
        layer.weight_scale = layer.weight_scale[:0]

    def apply(self, layer, x, bias):
        w4 = getattr(layer, "_w4", None)
        if w4 is not None:
            from ..ops import cuda as K

            return K.gemm_w4a16(_dequant_input(x, layer._compute_dtype), w4[0], w4[1], None, w4[2], 16, True, bias)
        return ops.gemm(_dequant_input(x, layer._dense.dtype), layer._dense, bias)

    def init_dummy(self, layer, gen, std=0.02):
        n, k2 = layer.weight_packed.shape
        w = _randn((n, k2 * 2), gen, std, layer.weight_packed.device)
        layer.weight_packed, layer.weight_scale, layer.weight_global_scale = nv_codec.quantize_nvfp4(w)


class Int4Method(LinearMethod):
    """AWQ / GPTQ / compressed-tensors int4, converted to the canonical (codes, scales, zeros) form
    after loading (python/minisgl/quant/kernels.py:255-346). On the GPU the codes are re-packed two
    per byte and stay 4-bit in HBM; the GEMM expands them tile by tile (W4A16: 16-bit activations,
    ``(code - zero) * scale`` exact). The CPU oracle path and odd shapes expand once at load."""

    def __init__(self, scheme: QuantScheme) -> None:
        self.scheme = scheme

    def create_weights(self, n, k, dtype, device):
        g, fmt = self.scheme.group_size, self.scheme.fmt
        e = lambda shape, dt: torch.empty(shape, dtype=dt, device=device)
        if fmt == "awq":
            return {"qweight": e((k, n // 8), torch.int32), "scales": e((k // g, n), torch.float16),
                    "qzeros": e((k // g, n // 8), torch.int32)}
        if fmt == "gptq":
            return {"qweight": e((k // 8, n), torch.int32), "scales": e((k // g, n), torch.float16),
                    "qzeros": e((k // g, n // 8), torch.int32)}
        out = {"weight_packed": e((n, k // 8), torch.int32), "weight_scale": e((n, k // g), torch.float16)}
        if not self.scheme.symmetric:
            out["weight_zero_point"] = e((n // 8, k // g), torch.int32)
        return out

    def shard_dims(self):
        if self.scheme.fmt in ("awq", "gptq"):
            return {"qweight": (1, 0), "scales": (1, 0), "qzeros": (1, 0)}
        return {"weight_packed": (0, 1), "weight_scale": (0, 1), "weight_zero_point": (0, 1)}

    def process_after_load(self, layer):
        fmt = self.scheme.fmt
        if fmt == "awq":
            c, s, z = int4_codec.awq_to_canonical(layer.qweight, layer.scales,
                                                  None if self.scheme.symmetric else layer.qzeros)
        elif fmt == "gptq":
            c, s, z = int4_codec.gptq_to_canonical(layer.qweight, layer.scales, layer.qzeros,
                                                   self.scheme.symmetric)
        else:
            c, s, z = int4_codec.ct_to_canonical(layer.weight_packed, layer.weight_scale,
                                                 getattr(layer, "weight_zero_point", None),
                                                 getattr(layer, "_ct_convention", None))
        n, k = c.shape
        group = k // s.shape[1]
        if _w4_native_ok(n, k, group, c.device) and layer._compute_dtype in (torch.bfloat16, torch.float16):
            packed = (c[:, 0::2] | (c[:, 1::2] << 4)).to(torch.uint8).contiguous()
            layer._w4 = (packed, s.float().t().contiguous(), z.float().t().contiguous(), group)
        else:
            layer._dense = int4_codec.dequant_int4(c, s, z).to(layer._compute_dtype)
        for name in ("qweight", "scales", "qzeros", "weight_packed", "weight_scale", "weight_zero_point"):
            if hasattr(layer, name):
                setattr(layer, name, getattr(layer, name)[:0])

    def apply(self, layer, x, bias):
        w4 = getattr(layer, "_w4", None)
        if w4 is not None:
            from ..ops import cuda as K

            return K.gemm_w4a16(_dequant_input(x, layer._compute_dtype), w4[0], w4[1], w4[2], None, w4[3], False, bias)
        return ops.gemm(_dequant_input(x, layer._dense.dtype), layer._dense, bias)

    def init_dummy(self, layer, gen, std=0.02):
        fmt = self.scheme.fmt
        if fmt in ("awq", "gptq"):
            k = layer.qweight.shape[0] * (1 if fmt == "awq" else 8)
            n = layer.qweight.shape[1] * (8 if fmt == "awq" else 1)
        else:
            n, k = layer.weight_packed.shape[0], layer.weight_packed.shape[1] * 8
        dev = next(iter(vars(layer).values())).device if False else None
        w = _randn((n, k), gen, std, "cpu")
        c, s, z = int4_codec.quantize_int4(w, self.scheme.group_size)
        tgt = layer.qweight.device if fmt in ("awq", "gptq") else layer.weight_packed.device
        if fmt == "awq":
            layer.qweight, layer.scales, layer.qzeros = (t.to(tgt) for t in int4_codec.pack_awq(c, s, z))
        elif fmt == "gptq":
            layer.qweight, layer.scales, layer.qzeros = (t.to(tgt) for t in int4_codec.pack_gptq(c, s, z))
        else:
            p, sc = int4_codec.pack_ct(c, s)
            layer.weight_packed, layer.weight_scale = p.to(tgt), sc.to(tgt)
            layer._ct_convention = "offset"


def make_linear_method(scheme: Optional[QuantScheme]) -> LinearMethod:
    name = scheme.name if scheme is not None else SCHEME_NONE
    if name == SCHEME_NONE:
        return UnquantizedMethod()
    if name == SCHEME_FP8_CHANNEL:
        return Fp8ChannelMethod()
    if name == SCHEME_FP8_TENSOR:
        return Fp8ChannelMethod(per_tensor=True)
    if name == SCHEME_FP8_BLOCK:
        return Fp8BlockMethod(scheme.block)
    if name == SCHEME_MXFP4:
        return MxFp4Method()
    if name == SCHEME_NVFP4:
        return NvFp4Method(scheme.global_scale_divides)
    if name == SCHEME_INT4:
        return Int4Method(scheme)
    raise ValueError(f"no linear method for scheme {name!r}")
