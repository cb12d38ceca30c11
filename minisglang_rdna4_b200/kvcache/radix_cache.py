"""Page-aligned radix tree over token ids with reference-count locking and LRU eviction.

Behaviour matches python/minisgl/kvcache/radix_cache.py:119-423: children are keyed by the
tokens of their first page; a match is aligned down to whole pages; a partial match splits
the node; locking a handle pins every node from it to the root and moves its pages from the
evictable to the protected count; eviction pops least-recently-used unlocked leaves from a
lazy heap and re-queues a parent that becomes a leaf.

The stored unit is a page id (one per ``page_size`` tokens). The common-prefix scan between
a query and a node key runs in the native host library when it is built.
"""
from __future__ import annotations

import heapq
import collections
import itertools
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .base import BaseCacheHandle, BasePrefixCache, SizeInfo
from ..ops.host import common_prefix_len


class RadixNode:
    __slots__ = ("key", "pages", "children", "parent", "ref", "stamp", "uid", "snap")
    _uids = itertools.count()

    def __init__(self, key: np.ndarray, pages: np.ndarray, parent: Optional["RadixNode"]) -> None:
        self.key = key          # int32 tokens, length = len(pages) * page_size
        self.pages = pages      # int32 page ids
        self.children: Dict[bytes, RadixNode] = {}
        self.parent = parent
        self.ref = 0
        self.stamp = time.monotonic_ns()
        self.uid = next(RadixNode._uids)
        self.snap: Optional[int] = None   # id of a recurrent-state snapshot taken exactly at this node's end

    @property
    def is_leaf(self) -> bool:
        return not self.children

    @property
    def is_root(self) -> bool:
        return self.parent is None


@dataclass
class RadixHandle(BaseCacheHandle):
    node: RadixNode = None  # type: ignore[assignment]
    snap: Optional[int] = None      # recurrent-state snapshot to restore for this prefix


class RadixPrefixCache(BasePrefixCache):
    def __init__(self, page_size: int) -> None:
        self.page_size = page_size
        self.reset()

    # ------------------------------------------------------------------ helpers
    def reset(self) -> None:
        empty = np.empty(0, dtype=np.int32)
        self.root = RadixNode(empty, empty, None)
        self.root.ref = 1  # never evicted
        self._evictable = 0
        self._protected = 0
        self._heap: List[Tuple[int, int, RadixNode]] = []

    def _child_key(self, tokens: np.ndarray) -> bytes:
        return tokens[: self.page_size].tobytes()

    @staticmethod
    def _as_np(ids) -> np.ndarray:
        if isinstance(ids, torch.Tensor):
            return ids.detach().to(torch.int32).numpy() if ids.dtype != torch.int32 else ids.numpy()
        return np.asarray(ids, dtype=np.int32)

    def _split(self, node: RadixNode, pages_kept: int) -> RadixNode:
        """Split ``node`` after ``pages_kept`` pages; returns the new upper node."""
        ps = self.page_size
        assert 0 < pages_kept < len(node.pages)
        upper = RadixNode(node.key[: pages_kept * ps], node.pages[:pages_kept], node.parent)
        upper.ref = node.ref
        upper.stamp = node.stamp
        assert node.parent is not None
        node.parent.children[self._child_key(upper.key)] = upper
        node.key = node.key[pages_kept * ps :]
        node.pages = node.pages[pages_kept:]
        node.parent = upper
        upper.children[self._child_key(node.key)] = node
        return upper

    def _walk(self, ids: np.ndarray) -> Tuple[RadixNode, int]:
        """Descend as far as ``ids`` matches; returns (deepest fully matched node, tokens)."""
        ps = self.page_size
        node, matched = self.root, 0
        total = (len(ids) // ps) * ps
        now = time.monotonic_ns()
        while matched < total:
            child = node.children.get(ids[matched : matched + ps].tobytes())
            if child is None:
                break
            limit = min(len(child.key), total - matched)
            same = common_prefix_len(child.key, ids[matched:], limit)
            same = (same // ps) * ps
            if same == 0:  # pragma: no cover - first page matched by construction
                break
            if same < len(child.key):
                child = self._split(child, same // ps)
            child.stamp = now
            node, matched = child, matched + same
            if same < limit:
                break
        return node, matched

    # ------------------------------------------------------------------ interface
    def match_prefix(self, input_ids: torch.Tensor) -> Tuple[RadixHandle, torch.Tensor]:
        ids = self._as_np(input_ids)
        node, matched = self._walk(ids)
        pages: List[np.ndarray] = []
        cur = node
        while not cur.is_root:
            pages.append(cur.pages)
            cur = cur.parent  # type: ignore[assignment]
        pages.reverse()
        flat = np.concatenate(pages) if pages else np.empty(0, dtype=np.int32)
        return RadixHandle(matched, node), torch.from_numpy(flat.copy())

    def lock_handle(self, handle: BaseCacheHandle, unlock: bool = False) -> None:
        assert isinstance(handle, RadixHandle)
        node = handle.node
        while not node.is_root:
            if unlock:
                node.ref -= 1
                assert node.ref >= 0, "radix node unlocked more often than locked"
                if node.ref == 0:
                    self._protected -= len(node.pages)
                    self._evictable += len(node.pages)
                    if node.is_leaf:
                        heapq.heappush(self._heap, (node.stamp, node.uid, node))
            else:
                if node.ref == 0:
                    self._evictable -= len(node.pages)
                    self._protected += len(node.pages)
                node.ref += 1
            node = node.parent  # type: ignore[assignment]

    def insert_prefix(self, input_ids: torch.Tensor, page_ids: torch.Tensor) -> int:
        ps = self.page_size
        ids = self._as_np(input_ids)
        n_tokens = (len(ids) // ps) * ps
        ids = ids[:n_tokens]
        pages = self._as_np(page_ids)[: n_tokens // ps]
        assert len(pages) * ps == n_tokens
        node, matched = self._walk(ids)
        if matched < n_tokens:
            new = RadixNode(ids[matched:].copy(), pages[matched // ps :].copy(), node)
            node.children[self._child_key(new.key)] = new
            self._evictable += len(new.pages)
            heapq.heappush(self._heap, (new.stamp, new.uid, new))
        return matched

    def evict(self, num_pages: int) -> torch.Tensor:
        if num_pages <= 0:
            return torch.empty(0, dtype=torch.int32)
        if num_pages > self._evictable:
            raise RuntimeError(f"cannot evict {num_pages} pages: only {self._evictable} are evictable")
        freed: List[np.ndarray] = []
        got = 0
        while got < num_pages:
            if not self._heap:
                self._rebuild_heap()
                if not self._heap:  # pragma: no cover - guarded by the size check above
                    raise RuntimeError("eviction heap is empty although pages are evictable")
            stamp, _, node = heapq.heappop(self._heap)
            # lazy heap: skip entries that are stale, locked, interior or already removed
            if node.parent is None or node.ref != 0 or not node.is_leaf or node.stamp != stamp:
                if node.parent is not None and node.ref == 0 and node.is_leaf and node.stamp != stamp:
                    heapq.heappush(self._heap, (node.stamp, node.uid, node))
                continue
            if node.parent.children.get(self._child_key(node.key)) is not node:
                continue
            del node.parent.children[self._child_key(node.key)]
            if node.snap is not None:
                self._drop_snapshot(node)
            freed.append(node.pages)
            got += len(node.pages)
            self._evictable -= len(node.pages)
            parent = node.parent
            node.parent = None
            if not parent.is_root and parent.is_leaf and parent.ref == 0:
                heapq.heappush(self._heap, (parent.stamp, parent.uid, parent))
        return torch.from_numpy(np.concatenate(freed))

    def _drop_snapshot(self, node: RadixNode) -> None:
        node.snap = None

    def _rebuild_heap(self) -> None:
        self._heap = []
        stack = [self.root]
        while stack:
            node = stack.pop()
            stack.extend(node.children.values())
            if not node.is_root and node.is_leaf and node.ref == 0:
                self._heap.append((node.stamp, node.uid, node))
        heapq.heapify(self._heap)

    @property
    def size_info(self) -> SizeInfo:
        return SizeInfo(self._evictable, self._protected)

    def check_integrity(self) -> None:
        evictable = protected = 0
        seen_pages = set()
        stack = [self.root]
        while stack:
            node = stack.pop()
            for key, child in node.children.items():
                assert child.parent is node
                assert key == self._child_key(child.key)
                assert len(child.key) == len(child.pages) * self.page_size
                assert child.ref <= node.ref or node.is_root, "child pinned more than its parent"
                stack.append(child)
            if node.is_root:
                continue
            assert len(node.pages) > 0
            for p in node.pages.tolist():
                assert p not in seen_pages, f"page {p} owned by two radix nodes"
                seen_pages.add(p)
            if node.ref == 0:
                evictable += len(node.pages)
            else:
                protected += len(node.pages)
        assert evictable == self._evictable, (evictable, self._evictable)
        assert protected == self._protected, (protected, self._protected)


class SnapshotRadixCache(RadixPrefixCache):
    """Prefix cache for models with recurrent layers (gated delta net, Mamba-2). Their per-request
    state is a running summary that cannot be cut at an arbitrary length, so a cached prefix is
    only reusable up to a boundary at which a snapshot of the state was taken. Nodes whose end
    coincides with such a boundary carry the snapshot's id; ``match_prefix`` returns the deepest
    matched boundary that has one, and the K/V pages of the attention layers up to it
    (python/minisgl/kvcache/radix_cache.py:119-423, python/minisgl/kvcache/composite_state.py:24).

    ``on_drop(id)`` is called when a snapshot leaves the cache (its node was evicted, replaced, or the
    ``capacity`` was reached and it was the least recently used)."""

    def __init__(self, page_size: int, capacity: int = 64, on_drop=None) -> None:
        self.capacity = max(int(capacity), 1)
        self.on_drop = on_drop
        self._lru: "collections.OrderedDict[int, RadixNode]" = collections.OrderedDict()
        super().__init__(page_size)

    def reset(self) -> None:
        for key in list(getattr(self, "_lru", {})):
            if self.on_drop is not None:
                self.on_drop(key)
        self._lru = collections.OrderedDict()
        super().reset()

    def _drop_snapshot(self, node: RadixNode) -> None:
        key, node.snap = node.snap, None
        if key is not None and self._lru.pop(key, None) is not None and self.on_drop is not None:
            self.on_drop(key)

    def match_prefix(self, input_ids: torch.Tensor) -> Tuple[RadixHandle, torch.Tensor]:
        ids = self._as_np(input_ids)
        node, matched = self._walk(ids)
        while not node.is_root and node.snap is None:      # back up to a boundary whose state is known
            matched -= len(node.key)
            node = node.parent  # type: ignore[assignment]
        pages: List[np.ndarray] = []
        cur = node
        while not cur.is_root:
            pages.append(cur.pages)
            cur = cur.parent  # type: ignore[assignment]
        pages.reverse()
        flat = np.concatenate(pages) if pages else np.empty(0, dtype=np.int32)
        if node.snap is not None:
            self._lru.move_to_end(node.snap)
        return RadixHandle(matched, node, node.snap), torch.from_numpy(flat.copy())

    def attach_snapshot(self, input_ids: torch.Tensor, length: int, key: int) -> bool:
        """Mark the cached prefix of exactly ``length`` tokens (a page multiple) with snapshot ``key``.
        False when that prefix is not in the cache; the caller then drops the snapshot."""
        if length <= 0 or length % self.page_size:
            return False
        ids = self._as_np(input_ids)[:length]
        if len(ids) < length:
            return False
        node, matched = self._walk(ids)        # splits the node that spans the boundary
        if matched != length or node.is_root:
            return False
        if node.snap is not None:
            self._drop_snapshot(node)
        node.snap = key
        self._lru[key] = node
        while len(self._lru) > self.capacity:
            _old, victim = next(iter(self._lru.items()))
            self._drop_snapshot(victim)
        return True

    @property
    def num_snapshots(self) -> int:
        return len(self._lru)
