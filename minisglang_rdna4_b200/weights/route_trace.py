"""Expert routing trace (python/minisgl/weights/route_trace.py:167): per MoE layer, how often
each expert was routed to. The host tier records into it on every step; the counts seed the
residency cache at the next boot (hot experts are copied in before the first request) and tell an
operator how skewed the routing of a workload is."""
from __future__ import annotations

import json
from typing import Dict, Iterable, List

import numpy as np


class RouteTrace:
    def __init__(self, num_experts: int) -> None:
        self.num_experts = num_experts
        self.counts: Dict[int, np.ndarray] = {}
        self.steps = 0

    def record(self, layer: int, expert_ids: Iterable[int]) -> None:
        c = self.counts.get(layer)
        if c is None:
            c = self.counts[layer] = np.zeros(self.num_experts, dtype=np.int64)
        ids = np.asarray(list(expert_ids) if not isinstance(expert_ids, np.ndarray) else expert_ids, dtype=np.int64)
        ids = ids[(ids >= 0) & (ids < self.num_experts)]
        np.add.at(c, ids, 1)
        self.steps += 1

    def hottest(self, layer: int, n: int) -> List[int]:
        c = self.counts.get(layer)
        if c is None:
            return []
        order = np.argsort(-c, kind="stable")
        return [int(e) for e in order[:n] if c[e] > 0]

    def skew(self, layer: int) -> float:
        """Share of the routed tokens that went to the top 10 % of the experts."""
        c = self.counts.get(layer)
        if c is None or c.sum() == 0:
            return 0.0
        top = max(1, self.num_experts // 10)
        return float(np.sort(c)[::-1][:top].sum() / c.sum())

    def save(self, path: str) -> None:
        with open(path, "w") as fh:
            json.dump({"num_experts": self.num_experts, "steps": self.steps,
                       "counts": {str(k): v.tolist() for k, v in self.counts.items()}}, fh)

    @classmethod
    def load(cls, path: str) -> "RouteTrace":
        with open(path) as fh:
            d = json.load(fh)
        t = cls(int(d["num_experts"]))
        t.steps = int(d.get("steps", 0))
        t.counts = {int(k): np.asarray(v, dtype=np.int64) for k, v in d["counts"].items()}
        return t
