"""Boot timeline (python/minisgl/weights/boot_timeline.py:222): wall-clock stamps of the stages
between process start and "engine ready", printed as one table so that a slow boot points at its
stage (weight load, offload bind, KV allocation, graph capture) without a profiler."""
from __future__ import annotations

import time
from typing import List, Tuple


class BootTimeline:
    def __init__(self, clock=time.perf_counter) -> None:
        self._clock = clock
        self._t0 = clock()
        self._last = self._t0
        self.stages: List[Tuple[str, float]] = []

    def mark(self, stage: str) -> float:
        """Close the stage that just ran; returns its duration in seconds."""
        now = self._clock()
        dt = now - self._last
        self._last = now
        self.stages.append((stage, dt))
        return dt

    @property
    def total(self) -> float:
        return self._last - self._t0

    def render(self) -> str:
        if not self.stages:
            return "boot: no stages recorded"
        width = max(len(s) for s, _ in self.stages)
        lines = [f"boot timeline ({self.total:.2f} s)"]
        for stage, dt in self.stages:
            share = 100.0 * dt / self.total if self.total > 0 else 0.0
            lines.append(f"  {stage:<{width}}  {dt:8.3f} s  {share:5.1f} %")
        return "\n".join(lines)
