"""Gated activations (SwiGLU / GeGLU; python/minisgl/layers/activation.py:25-64)."""
from __future__ import annotations

from typing import Union

import torch

from .. import ops
from ..quant.method import ActQ


class GatedActivation:
    def __init__(self, kind: str = "silu") -> None:
        if kind not in ("silu", "gelu", "gelu_pytorch_tanh", "gelu_tanh"):
            raise ValueError(f"unsupported gated activation {kind!r}")
        self.kind = kind

    def __call__(self, x: torch.Tensor, quant: bool = False) -> Union[torch.Tensor, ActQ]:
        if self.kind == "silu":
            if quant:
                return ActQ(*ops.silu_and_mul_quant(x))
            return ops.silu_and_mul(x)
        y = ops.gelu_and_mul(x, tanh=self.kind != "gelu")
        return ActQ(*ops.per_token_quant_fp8(y)) if quant else y
