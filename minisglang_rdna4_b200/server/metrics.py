"""Prometheus text exposition, hand-rolled (python/minisgl/server/metrics.py:31-39,122-376):
request counters, TTFT / TPOT / end-to-end latency histograms, and gauges relayed from the
schedulers (running, waiting, KV usage, prefix-cache hits, speculative-decode counters)."""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional, Tuple

_TTFT_BUCKETS = (0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0)
_TPOT_BUCKETS = (0.001, 0.0025, 0.005, 0.0075, 0.01, 0.015, 0.02, 0.03, 0.05, 0.1, 0.25, 1.0)
_E2E_BUCKETS = (0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0, 120.0, 300.0)


class Histogram:
    def __init__(self, name: str, doc: str, buckets: Tuple[float, ...]) -> None:
        self.name, self.doc, self.buckets = name, doc, buckets
        self.counts = [0] * (len(buckets) + 1)
        self.total = 0.0
        self.n = 0

    def observe(self, v: float) -> None:
        self.total += v
        self.n += 1
        for i, b in enumerate(self.buckets):
            if v <= b:
                self.counts[i] += 1
                return
        self.counts[-1] += 1

    def render(self, prefix: str) -> List[str]:
        full = prefix + self.name
        out = [f"# HELP {full} {self.doc}", f"# TYPE {full} histogram"]
        acc = 0
        for b, c in zip(self.buckets, self.counts):
            acc += c
            out.append(f'{full}_bucket{{le="{b}"}} {acc}')
        out.append(f'{full}_bucket{{le="+Inf"}} {self.n}')
        out.append(f"{full}_sum {self.total}")
        out.append(f"{full}_count {self.n}")
        return out


class FrontendMetrics:
    PREFIX = "minisgl_"

    def __init__(self, model_name: str = "model") -> None:
        self.model = model_name
        self.lock = threading.Lock()
        self.counters: Dict[str, float] = {
            "requests_total": 0, "requests_finished_total": 0, "requests_aborted_total": 0,
            "requests_failed_total": 0, "prompt_tokens_total": 0, "generation_tokens_total": 0,
            "cached_prompt_tokens_total": 0,
        }
        self.ttft = Histogram("time_to_first_token_seconds", "time from request to first token", _TTFT_BUCKETS)
        self.tpot = Histogram("time_per_output_token_seconds", "mean inter-token latency of a request", _TPOT_BUCKETS)
        self.e2e = Histogram("e2e_request_latency_seconds", "request latency", _E2E_BUCKETS)
        self.scheduler: Dict[int, Dict[str, float]] = {}
        self._start: Dict[int, float] = {}
        self._first: Dict[int, float] = {}
        self._tokens: Dict[int, int] = {}

    # ---- request lifecycle ----
    def on_request(self, uid: int) -> None:
        with self.lock:
            self.counters["requests_total"] += 1
            self._start[uid] = time.monotonic()
            self._tokens[uid] = 0

    def on_token(self, uid: int, n: int = 1) -> None:
        now = time.monotonic()
        with self.lock:
            if uid not in self._start:
                return
            if uid not in self._first:
                self._first[uid] = now
                self.ttft.observe(now - self._start[uid])
            self._tokens[uid] = self._tokens.get(uid, 0) + n
            self.counters["generation_tokens_total"] += n

    def on_finish(self, uid: int, reason: Optional[str], prompt_tokens: int = 0, cached_tokens: int = 0) -> None:
        now = time.monotonic()
        with self.lock:
            start = self._start.pop(uid, None)
            first = self._first.pop(uid, None)
            n = self._tokens.pop(uid, 0)
            if start is None:
                return
            key = {"abort": "requests_aborted_total", "error": "requests_failed_total"}.get(
                reason or "", "requests_finished_total")
            self.counters[key] += 1
            self.counters["prompt_tokens_total"] += prompt_tokens
            self.counters["cached_prompt_tokens_total"] += cached_tokens
            self.e2e.observe(now - start)
            if first is not None and n > 1:
                self.tpot.observe((now - first) / (n - 1))

    def on_scheduler_stats(self, dp_rank: int, values: Dict[str, float]) -> None:
        with self.lock:
            self.scheduler[dp_rank] = dict(values)

    # ---- exposition ----
    def render(self) -> str:
        p = self.PREFIX
        lines: List[str] = []
        with self.lock:
            for name, val in sorted(self.counters.items()):
                lines += [f"# TYPE {p}{name} counter", f'{p}{name}{{model="{self.model}"}} {val}']
            for h in (self.ttft, self.tpot, self.e2e):
                lines += h.render(p)
            gauges = ("running", "waiting", "kv_tokens_used", "kv_tokens_total", "prefix_hit_tokens",
                      "prefix_query_tokens", "spec_drafted", "spec_accepted", "spec_emitted", "spec_steps",
                      "prefill_tokens", "decode_tokens", "steps")
            for g in gauges:
                rows = [(r, v[g]) for r, v in sorted(self.scheduler.items()) if g in v]
                if not rows:
                    continue
                lines.append(f"# TYPE {p}scheduler_{g} gauge")
                for r, v in rows:
                    lines.append(f'{p}scheduler_{g}{{dp_rank="{r}"}} {v}')
        return "\n".join(lines) + "\n"
