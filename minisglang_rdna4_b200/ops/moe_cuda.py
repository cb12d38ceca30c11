"""Mixture-of-experts ops on the GPU: routing and the expert MLPs.

Routing (softmax / sigmoid scores, optional selection bias, top-k, renormalise) and the
token→expert grouping run as one fused kernel when ``libmsgl_cuda`` exports it; the expert
MLPs run as grouped tcgen05 GEMMs over tokens sorted by expert (each expert's rows padded to
the 128-row tile), with SiLU·mul between them and the gate-weighted combine at the end.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import cuda as K
from . import ref


def moe_route(router_logits, top_k, renormalize, scoring="softmax", bias=None, scale=1.0):
    from ._lib import lib

    if hasattr(lib(), "msgl_moe_route") and bias is None:
        from .moe_kernels import moe_route as fused

        return fused(router_logits, top_k, renormalize, scoring, scale)
    return ref.moe_route(router_logits, top_k, renormalize, scoring, bias, scale)


def moe_forward(x, w13, w2, topk_w, topk_ids, expert_offset=0):
    from ._lib import lib

    if hasattr(lib(), "msgl_moe_align"):
        from .moe_kernels import moe_forward as fused

        return fused(x, w13, w2, topk_w, topk_ids, expert_offset)
    # per-expert loop on the dense tcgen05 GEMM (functional path)
    t, h = x.shape
    e_local = w13.shape[0]
    out = torch.zeros((t, h), dtype=torch.float32, device=x.device)
    for e in range(e_local):
        sel = topk_ids == (e + expert_offset)
        rows = sel.any(-1).nonzero().squeeze(-1)
        if rows.numel() == 0:
            continue
        wt = (topk_w * sel).sum(-1)[rows]
        hcur = K.gemm(x[rows].contiguous(), w13[e])
        act = K.act_and_mul(hcur)
        y = K.gemm(act, w2[e], None, torch.float32)
        out.index_add_(0, rows, y * wt[:, None])
    return out.to(x.dtype)
