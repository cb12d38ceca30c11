"""Prompt-lookup (n-gram) proposer (python/minisgl/spec/proposer.py:17,58-105): take the
longest suffix n-gram (from ``ngram_max`` down to ``ngram_min`` tokens) that occurred earlier
within the last 4096 tokens of the sequence, and propose the tokens that followed its most
recent earlier occurrence."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np

from ..core import Req
from .base import Proposer

LOOKBACK = 4096


def ngram_lookup(tokens: np.ndarray, k: int, n_max: int, n_min: int) -> List[int]:
    total = len(tokens)
    if k <= 0 or total < n_min + 1:
        return []
    window = tokens[max(0, total - LOOKBACK):]
    w = len(window)
    for n in range(min(n_max, w - 1), n_min - 1, -1):
        suffix = window[w - n:]
        # candidate starts: positions whose n tokens equal the suffix, excluding the suffix itself
        limit = w - n  # start index of the suffix
        if limit <= 0:
            continue
        hits = np.flatnonzero(window[:limit] == suffix[0])
        for start in hits[::-1]:
            if start + n > limit + n - 1 and start == limit:
                continue
            if np.array_equal(window[start:start + n], suffix):
                follow = window[start + n:start + n + k]
                if len(follow):
                    return follow.tolist()
    return []


def ngram_lookup_paths(tokens: np.ndarray, k: int, n_max: int, n_min: int, width: int) -> List[List[int]]:
    """Up to ``width`` distinct continuations of the longest matching suffix n-gram, most recent
    occurrence first: the candidates of a draft tree."""
    total = len(tokens)
    if k <= 0 or width <= 0 or total < n_min + 1:
        return []
    window = tokens[max(0, total - LOOKBACK):]
    w = len(window)
    for n in range(min(n_max, w - 1), n_min - 1, -1):
        suffix = window[w - n:]
        limit = w - n
        if limit <= 0:
            continue
        paths: List[List[int]] = []
        for start in np.flatnonzero(window[:limit] == suffix[0])[::-1]:
            if np.array_equal(window[start:start + n], suffix):
                follow = window[start + n:start + n + k].tolist()
                if follow and follow not in paths:
                    paths.append(follow)
                    if len(paths) == width:
                        break
        if paths:
            return paths
    return []


class NgramProposer(Proposer):
    name = "ngram"

    def __init__(self, num_draft: int, n_max: int = 3, n_min: int = 1, tree_width: int = 1) -> None:
        super().__init__(num_draft)
        self.n_max, self.n_min = n_max, n_min
        self.tree_width = tree_width

    def propose_paths(self, reqs: Sequence[Req]) -> List[List[List[int]]]:
        """Per request, up to ``tree_width`` candidate continuations (best first) for a draft tree."""
        return [ngram_lookup_paths(r.input_ids.numpy(), self.budget(r), self.n_max, self.n_min, self.tree_width)
                for r in reqs]

    def propose(self, reqs: Sequence[Req]) -> List[List[int]]:
        out = []
        for r in reqs:
            out.append(ngram_lookup(r.input_ids.numpy(), self.budget(r), self.n_max, self.n_min))
        return out
