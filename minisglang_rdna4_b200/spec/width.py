"""Adaptive verify width (python/minisgl/spec/width.py:141-260): keep an exponential moving
average of how many draft tokens are accepted and shrink or grow the number of draft rows
that are verified, so a proposer that keeps missing does not pay for wide verify batches."""
from __future__ import annotations


class AdaptiveWidth:
    def __init__(self, max_width: int, min_width: int = 1, alpha: float = 0.2) -> None:
        self.max_width, self.min_width, self.alpha = max_width, max(min_width, 1), alpha
        self.mean_accept = float(max_width) / 2
        self.steps = 0

    def update(self, accepted: float) -> None:
        self.steps += 1
        self.mean_accept = (1 - self.alpha) * self.mean_accept + self.alpha * accepted

    def choose(self) -> int:
        # verify about one token more than what is usually accepted
        want = int(self.mean_accept + 1.5)
        return max(self.min_width, min(self.max_width, want))
