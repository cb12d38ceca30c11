"""Draft token trees for tree-structured verification (python/minisgl/spec/ddtree.py,
spec/tidar_mask.py): several candidate continuations share one verify forward; every node
attends to the committed prefix and to its own ancestors through an additive mask, which is the
``mask`` operand of the general paged-attention kernel (``Batch.tree_mask``).

This module is the host-side geometry: building a tree from ranked candidates, the rows a verify
step feeds (tokens, positions, KV slots), the mask, greedy acceptance along the tree, and the KV
moves that make the accepted path contiguous afterwards. The speculative step of the scheduler
feeds linear drafts today; a proposer that emits trees plugs in through these helpers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class TokenTree:
    """Node 0 is the root: the request's last committed token. ``parent[i] < i`` for i > 0."""

    tokens: List[int]
    parent: List[int] = field(default_factory=lambda: [-1])

    def __post_init__(self) -> None:
        if len(self.tokens) != len(self.parent) or not self.tokens or self.parent[0] != -1:
            raise ValueError("a tree needs one parent entry per token and a root with parent -1")
        if any(not (0 <= p < i) for i, p in enumerate(self.parent) if i > 0):
            raise ValueError("parents must precede their children")

    def __len__(self) -> int:
        return len(self.tokens)

    @property
    def depth(self) -> List[int]:
        d = [0] * len(self.tokens)
        for i in range(1, len(self.tokens)):
            d[i] = d[self.parent[i]] + 1
        return d

    def children(self, node: int) -> List[int]:
        return [i for i, p in enumerate(self.parent) if p == node]

    def ancestors(self, node: int) -> List[int]:
        """The node itself and everything up to the root."""
        out = []
        while node >= 0:
            out.append(node)
            node = self.parent[node]
        return out

    @classmethod
    def from_paths(cls, root_token: int, paths: Sequence[Sequence[int]], max_nodes: int = 64) -> "TokenTree":
        """Merge candidate continuations (best first) into a prefix tree of at most ``max_nodes``
        nodes; shared prefixes become shared nodes."""
        tokens, parent = [int(root_token)], [-1]
        index: Dict[Tuple[int, int], int] = {}
        for path in paths:
            node = 0
            for t in path:
                key = (node, int(t))
                nxt = index.get(key)
                if nxt is None:
                    if len(tokens) >= max_nodes:
                        break
                    nxt = index[key] = len(tokens)
                    tokens.append(int(t))
                    parent.append(node)
                node = nxt
        return cls(tokens, parent)

    @classmethod
    def chain(cls, root_token: int, draft: Sequence[int]) -> "TokenTree":
        return cls([int(root_token)] + [int(t) for t in draft], [-1] + list(range(len(draft))))


def verify_rows(tree: TokenTree, prefix_len: int) -> Tuple[List[int], List[int], List[int]]:
    """``(tokens, positions, kv_slots)`` of the verify step. ``prefix_len`` counts the committed
    tokens before the root. A node's rotary position is its depth below the prefix; its K/V go to
    the scratch slot ``prefix_len + node index`` (node order, not depth: siblings need distinct
    slots)."""
    depth = tree.depth
    return list(tree.tokens), [prefix_len + d for d in depth], [prefix_len + i for i in range(len(tree))]


def tree_mask(tree: TokenTree, prefix_len: int, width: int, dtype=torch.float32) -> torch.Tensor:
    """Additive mask ``[nodes, width]`` over KV slots: 0 for the committed prefix and for the slots of
    the node's ancestors (itself included), -inf elsewhere."""
    n = len(tree)
    if width < prefix_len + n:
        raise ValueError("the mask must cover the prefix and every node's slot")
    m = torch.full((n, width), float("-inf"), dtype=dtype)
    m[:, :prefix_len] = 0.0
    for i in range(n):
        for a in tree.ancestors(i):
            m[i, prefix_len + a] = 0.0
    return m


def accept_greedy_tree(tree: TokenTree, target: Sequence[int]) -> Tuple[List[int], List[int]]:
    """``target[i]`` is the target model's arg-max after node i. Walk down from the root while some
    child carries the token the target wants; returns ``(emitted tokens, accepted node path)``.
    The emitted tokens are the accepted children plus the target's own token after the last
    accepted node (the bonus token), so at least one token is always emitted."""
    node, path, emitted = 0, [0], []
    while True:
        want = int(target[node])
        emitted.append(want)
        nxt = next((c for c in tree.children(node) if tree.tokens[c] == want), None)
        if nxt is None:
            return emitted, path
        node = nxt
        path.append(node)


def compaction_moves(path: Sequence[int], prefix_len: int) -> List[Tuple[int, int]]:
    """``(src_slot, dst_slot)`` copies that bring the accepted nodes' K/V to the positions they hold
    in the committed sequence. Node ``path[d]`` sits at slot ``prefix_len + path[d]`` and belongs at
    ``prefix_len + d``; since ``path[d] >= d`` the copies are safe in ascending order of depth."""
    return [(prefix_len + n, prefix_len + d) for d, n in enumerate(path) if n != d]


def apply_moves(k_rows: torch.Tensor, v_rows: torch.Tensor, moves: Sequence[Tuple[int, int]]) -> None:
    """In-place on ``[slots, ...]`` views of one request's K and V."""
    for src, dst in moves:
        k_rows[dst] = k_rows[src]
        v_rows[dst] = v_rows[src]
