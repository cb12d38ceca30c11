"""Draft trees from a block drafter's per-position distributions (python/minisgl/spec/ddtree.py:1-501).

A one-pass block drafter (TiDAR's self-drafting forward, DFlash) gives, for each of the next ``k`` positions,
a distribution that does not depend on what is chosen at the other positions. Instead of keeping only the
arg-max chain, the ``budget`` most probable PREFIXES under the product of those marginals are kept: a
prefix-closed set, i.e. a tree, which one verification forward scores with an ancestors-only mask.

Best-first enumeration: a prefix is (depth, rank chosen at each depth); its score is the sum of the chosen
log-probabilities. From a popped prefix the two ways to the next-best unseen prefixes are its next sibling
(the last rank + 1) and its first child (one more position at rank 0); both score no higher than the prefix
itself, so a heap pops prefixes in descending score and every popped prefix has its parent popped before it.
"""
from __future__ import annotations

import heapq
from typing import List, Sequence, Tuple


def build_draft_paths(topk_logp: Sequence[Sequence[float]], topk_ids: Sequence[Sequence[int]], budget: int
                      ) -> List[List[int]]:
    """``topk_logp[d][r]`` / ``topk_ids[d][r]``: log-probability and token of rank ``r`` (descending) at draft
    position ``d``. Returns up to ``budget`` token paths, best first, whose set is prefix-closed (every path's
    parent path is in the list before it)."""
    depth = len(topk_logp)
    if depth == 0 or budget <= 0:
        return []
    out: List[List[int]] = []
    # (-score, tie-break counter, ranks)
    heap: List[Tuple[float, int, Tuple[int, ...]]] = [(-float(topk_logp[0][0]), 0, (0,))]
    count = 1
    while heap and len(out) < budget:
        neg, _, ranks = heapq.heappop(heap)
        d = len(ranks)
        out.append([int(topk_ids[i][r]) for i, r in enumerate(ranks)])
        last = ranks[-1]
        if last + 1 < len(topk_logp[d - 1]):              # next sibling
            score = -neg - float(topk_logp[d - 1][last]) + float(topk_logp[d - 1][last + 1])
            heapq.heappush(heap, (-score, count, ranks[:-1] + (last + 1,)))
            count += 1
        if d < depth:                                       # first child
            heapq.heappush(heap, (neg - float(topk_logp[d][0]), count, ranks + (0,)))
            count += 1
    return out
