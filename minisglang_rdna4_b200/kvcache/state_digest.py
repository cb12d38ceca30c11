"""Exact per-layer digests of the state a prefill leaves behind; a diagnostic
(python/minisgl/kvcache/state_digest.py:1-210).

A prefix-reuse or chunking bug shows up as text that differs, after every layer and the sampler
have amplified it. What prefix reuse actually promises is narrower and checkable: the K/V (and,
for hybrid models, the recurrent state) that a prefill leaves in the pools is what a cold prefill
of the same tokens leaves. So the digest is taken of the state itself: SHA-256 over the raw bytes
of every attention layer's K and V, in segments of ``SEG`` absolute positions, and of every
recurrent layer's convolution tail and state matrix. Segments by absolute position separate the
two failure stories of a reused prefill: a difference only in the span the forward just computed
blames the extend, a difference inside the reused span blames what the cache handed over.

Off unless ``MSGL_STATE_DIGEST=1``: it copies a request's whole K/V to the host and hashes it.
"""
from __future__ import annotations

import hashlib
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..env import ENV
from ..utils import init_logger

logger = init_logger(__name__)

SEG = 256
Key = Tuple[str, int, int]          # (pool, layer, segment)


def enabled() -> bool:
    return bool(ENV.STATE_DIGEST.value)


def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()[:16]


def kv_digests(pool, pages: np.ndarray, length: int, name: str = "kv") -> Dict[Key, str]:
    """``pages``: the request's page ids in position order. One digest per (layer, segment of SEG
    positions) over K then V of positions ``[0, length)``."""
    out: Dict[Key, str] = {}
    ps = pool.page_size
    n_pages = (length + ps - 1) // ps
    idx = torch.as_tensor(np.asarray(pages[:n_pages], dtype=np.int64), device=pool.device)
    for layer in range(pool.num_layers):
        # [pages, heads, page, dim] -> [positions, heads, dim]
        k = pool.k_cache(layer)[idx].permute(0, 2, 1, 3).reshape(n_pages * ps, -1)[:length]
        v = pool.v_cache(layer)[idx].permute(0, 2, 1, 3).reshape(n_pages * ps, -1)[:length]
        for seg, start in enumerate(range(0, length, SEG)):
            out[(name, layer, seg)] = _sha(torch.stack([k[start:start + SEG], v[start:start + SEG]]))
    return out


def recurrent_digests(state, slot: int) -> Dict[Key, str]:
    out: Dict[Key, str] = {}
    for layer in range(state.num_layers):
        out[("conv", layer, 0)] = _sha(state.conv[layer, slot])
        out[("state", layer, 0)] = _sha(state.ssm[layer, slot])
    return out


def request_digests(sched, req) -> Dict[Key, str]:
    """Everything the engine holds for ``req`` after a step: K/V of ``[0, cached_len)``, recurrent state."""
    eng = sched.engine
    if eng.stream is not None:
        eng.stream.synchronize()
    out = kv_digests(eng.kv_cache, sched.cache.page_table[req.table_idx], int(req.cached_len))
    if eng.gdn_state is not None:
        out.update(recurrent_digests(eng.gdn_state, req.table_idx))
    return out


def first_difference(a: Dict[Key, str], b: Dict[Key, str]) -> Optional[Key]:
    """The first (pool, layer, segment) on which two digests disagree, layers before segments."""
    for key in sorted(set(a) | set(b), key=lambda k: (k[0], k[1], k[2])):
        if a.get(key) != b.get(key):
            return key
    return None


def log_request(sched, req, what: str) -> Dict[Key, str]:
    d = request_digests(sched, req)
    whole = hashlib.sha256("".join(f"{k}{v}" for k, v in sorted(d.items())).encode()).hexdigest()[:16]
    logger.info("state-digest %s uid=%d len=%d cached_at_admission=%d all=%s", what, req.uid, int(req.cached_len),
                sched.prefix_len.get(req.uid, 0), whole)
    for (pool, layer, seg), h in sorted(d.items()):
        logger.debug("state-digest uid=%d %s layer=%d seg=%d %s", req.uid, pool, layer, seg, h)
    sched.last_state_digests[req.uid] = d
    return d
