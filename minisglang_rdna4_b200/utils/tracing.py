"""Opt-in tracing of the serving loop, switched on by environment variables.

* ``MSGL_PROFILE=<path>``: a ``torch.profiler`` window (CPU + CUDA activities) that opens after
  ``MSGL_PROFILE_SKIP`` forward steps, covers ``MSGL_PROFILE_STEPS`` steps and writes a chrome
  trace to ``<path>`` (rank r > 0 appends ``.rank<r>``). The reference wraps the same window
  around its scheduler loop (python/minisgl/scheduler/scheduler.py, ``MINISGL_PROFILE*``).
* ``MSGL_HOSTPROF=1``: host-side stage breakdown of the loop (receive, schedule, plan + launch,
  result processing); one summary line every 256 steps and at exit.
* ``MSGL_GRAPH_TIMING=1``: CUDA events around every graph replay (engine/graph.py) with the
  mean per bucket printed at exit.
* ``MSGL_LOG_REQUESTS=1``: one log line per admitted and per finished request.

Everything here is a no-op when the variables are unset; nothing on the hot path reads the
environment more than once.
"""
from __future__ import annotations

import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Dict, Optional

from ..env import ENV
from . import init_logger

logger = init_logger(__name__)


class StepProfiler:
    """``torch.profiler`` window over a range of forward steps."""

    def __init__(self, rank: int = 0) -> None:
        path = ENV.PROFILE.value
        self.path = (path if rank == 0 else f"{path}.rank{rank}") if path else ""
        self.skip = max(0, ENV.PROFILE_SKIP.value)
        self.steps = max(1, ENV.PROFILE_STEPS.value)
        self._prof = None
        self._done = not self.path

    def on_step(self, step: int) -> None:
        """Call once per loop iteration with the number of forward steps finished so far."""
        if self._done:
            return
        if self._prof is None and step >= self.skip:
            import torch

            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts, record_shapes=False)
            self._prof.__enter__()
            self._start = step
        elif self._prof is not None and step >= self._start + self.steps:
            self.close()

    def close(self) -> None:
        if self._prof is not None:
            self._prof.__exit__(None, None, None)
            try:
                self._prof.export_chrome_trace(self.path)
                logger.info("profiler trace written to %s", self.path)
            except Exception as exc:  # pragma: no cover - disk errors
                logger.warning("could not write profiler trace: %s", exc)
            self._prof = None
        self._done = True


class HostStages:
    """Wall-clock per stage of the scheduler loop."""

    def __init__(self) -> None:
        self.enabled = bool(ENV.HOSTPROF.value)
        self.total: Dict[str, float] = defaultdict(float)
        self.count: Dict[str, int] = defaultdict(int)
        self._iters = 0

    @contextmanager
    def stage(self, name: str):
        if not self.enabled:
            yield
            return
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.total[name] += time.perf_counter() - t0
            self.count[name] += 1

    def tick(self) -> None:
        if not self.enabled:
            return
        self._iters += 1
        if self._iters % 256 == 0:
            logger.info("hostprof %s", self.summary())

    def summary(self) -> str:
        parts = []
        for name in sorted(self.total, key=self.total.get, reverse=True):
            n = max(1, self.count[name])
            parts.append(f"{name}={1e3 * self.total[name] / n:.3f}ms x{self.count[name]}")
        return " ".join(parts) if parts else "(no samples)"


class GraphTimer:
    """CUDA-event timing of graph replays, keyed by bucket size."""

    def __init__(self) -> None:
        self.enabled = bool(ENV.GRAPH_TIMING.value)
        self._pending = []
        self.ms: Dict[int, float] = defaultdict(float)
        self.n: Dict[int, int] = defaultdict(int)

    def begin(self, bucket: int):
        if not self.enabled:
            return None
        import torch

        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        return (bucket, s, e)

    def end(self, token) -> None:
        if token is None:
            return
        token[2].record()
        self._pending.append(token)
        if len(self._pending) >= 64:
            self.flush()

    def flush(self) -> None:
        for bucket, s, e in self._pending:
            e.synchronize()
            self.ms[bucket] += s.elapsed_time(e)
            self.n[bucket] += 1
        self._pending.clear()

    def summary(self) -> str:
        self.flush()
        return " ".join(f"bs{b}={self.ms[b] / self.n[b]:.3f}ms x{self.n[b]}" for b in sorted(self.n))


def log_request(event: str, uid: int, **fields) -> None:
    if ENV.LOG_REQUESTS.value:
        logger.info("req %s uid=%d %s", event, uid, " ".join(f"{k}={v}" for k, v in fields.items()))
