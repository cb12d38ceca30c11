"""Draft acceptance.

Greedy verification is exact: accept the longest prefix of the draft for which the target's
arg-max at the preceding row equals the draft token, then emit the target token at the first
mismatch (or the bonus token after a fully accepted draft). The emitted tokens are by
construction the tokens plain greedy decoding would have produced
(python/minisgl/spec/accept.py:15-44). ``accept_greedy_device`` does the same for a whole
batch on the device without a host round trip per request
(python/minisgl/spec/accept_gpu.py:110-330); rejection sampling keeps the target distribution
for sampled requests (python/minisgl/spec/sampling.py:37-180).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def accept_greedy(target: Sequence[int], draft: Sequence[int]) -> List[int]:
    """``target`` has ``len(draft) + 1`` entries: row i is the arg-max after consuming the
    last committed token and draft[:i]. Returns the emitted tokens (1 ..= len(draft)+1)."""
    n = 0
    while n < len(draft) and int(target[n]) == int(draft[n]):
        n += 1
    return [int(t) for t in target[: n + 1]]


def accept_greedy_device(target: torch.Tensor, drafts: torch.Tensor, cu: torch.Tensor,
                         draft_lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Batched greedy acceptance on the device.

    ``target`` ``[T]`` arg-max of every verify row (packed, request b owns rows
    ``cu[b]:cu[b+1]`` = 1 + K_b rows); ``drafts`` ``[B, Kmax]`` padded with -1. Returns
    ``(n_emit [B], emitted [B, Kmax+1])`` where row b holds ``n_emit[b]`` valid tokens."""
    b, kmax = drafts.shape
    idx = cu[:-1].long()[:, None] + torch.arange(kmax + 1, device=target.device)[None, :]
    idx = idx.clamp_max(target.numel() - 1)
    tgt = target[idx]                                     # [B, Kmax+1]
    valid = torch.arange(kmax, device=target.device)[None, :] < draft_lens[:, None]
    match = (tgt[:, :kmax] == drafts) & valid
    accepted = match.long().cumprod(dim=1).sum(dim=1)     # length of the matching prefix
    n_emit = accepted + 1
    return n_emit.to(torch.int32), tgt


def eos_truncate(emitted: List[int], eos_ids, ignore_eos: bool) -> Tuple[List[int], bool]:
    """Cut the emitted run after the first end-of-sequence token."""
    if ignore_eos:
        return emitted, False
    for i, t in enumerate(emitted):
        if t in eos_ids:
            return emitted[: i + 1], True
    return emitted, False


def accept_rejection_sampling(target_probs: torch.Tensor, draft_probs: Optional[torch.Tensor],
                              draft: Sequence[int], generator: Optional[torch.Generator] = None) -> List[int]:
    """Speculative sampling for one request: draft token x_i is kept with probability
    ``min(1, p(x_i) / q(x_i))``; at the first rejection a token is drawn from
    ``norm(max(p - q, 0))``; after a fully accepted draft the bonus token is drawn from the
    last target row. ``draft_probs`` None means a deterministic proposer (q is a point mass)."""
    out: List[int] = []
    k = len(draft)
    for i in range(k):
        p = target_probs[i]
        x = int(draft[i])
        if draft_probs is None:
            q_x, q = 1.0, None
        else:
            q = draft_probs[i]
            q_x = float(q[x])
        u = float(torch.rand((), generator=generator, device="cpu"))
        if q_x > 0 and u < min(1.0, float(p[x]) / q_x):
            out.append(x)
            continue
        if q is None:
            resid = p.clone()
            resid[x] = 0.0
        else:
            resid = (p - q).clamp_min(0.0)
        if float(resid.sum()) <= 0:
            resid = p
        resid = resid / resid.sum()
        out.append(int(torch.multinomial(resid.cpu(), 1, generator=generator)))
        return out
    out.append(int(torch.multinomial(target_probs[k].cpu(), 1, generator=generator)))
    return out
