"""Token-sequence gates (python/minisgl/scheduler/think_gate.py:123 ToolCallGate, :252
ThinkGate).

``ThinkGate`` follows a request's reasoning span on token ids: while the span is open the
grammar of the request is held back; the span ends when the close delimiter (or a tool-call
opener) has been emitted; a budget forces the close delimiter out token by token when the
model keeps thinking past it. ``ToolCallGate`` suppresses the end-of-sequence token while a
tool call that the model opened has not been closed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence


def _ends_with(history: Sequence[int], pattern: Sequence[int]) -> bool:
    n = len(pattern)
    return n > 0 and len(history) >= n and list(history[-n:]) == list(pattern)


@dataclass
class ThinkGate:
    close_ids: List[int]                                  # token ids of the close delimiter
    release_patterns: List[List[int]] = field(default_factory=list)   # tool-call openers
    budget: int = 0                                       # 0 = unbounded
    span_open: bool = True                                # the prompt left the model inside the span
    released: bool = False
    thought: int = 0
    _forcing: int = 0                                     # index of the next forced close token
    _tail: List[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        if not self.span_open:
            self.released = True

    @property
    def grammar_active(self) -> bool:
        return self.released

    def forced_token(self) -> Optional[int]:
        """Token the sampler must emit next (budget exhausted), or None."""
        if self.released or self.budget <= 0 or not self.close_ids:
            return None
        if self._forcing > 0 or self.thought >= self.budget:
            return self.close_ids[self._forcing]
        return None

    def observe(self, token: int) -> None:
        if self.released:
            return
        self.thought += 1
        self._tail.append(int(token))
        keep = max([len(self.close_ids)] + [len(p) for p in self.release_patterns] + [1])
        if len(self._tail) > keep:
            del self._tail[: len(self._tail) - keep]
        if self._forcing > 0 or (self.budget > 0 and self.thought > self.budget):
            if self._forcing < len(self.close_ids) and token == self.close_ids[self._forcing]:
                self._forcing += 1
                if self._forcing == len(self.close_ids):
                    self.released = True
                return
        if _ends_with(self._tail, self.close_ids) or any(_ends_with(self._tail, p) for p in self.release_patterns):
            self.released = True


@dataclass
class ToolCallGate:
    openers: List[List[int]]
    closers: List[List[int]]
    open_calls: int = 0
    _tail: List[int] = field(default_factory=list)

    def observe(self, token: int) -> None:
        self._tail.append(int(token))
        keep = max([len(p) for p in self.openers + self.closers] + [1])
        if len(self._tail) > keep:
            del self._tail[: len(self._tail) - keep]
        if any(_ends_with(self._tail, p) for p in self.openers):
            self.open_calls += 1
        elif self.open_calls > 0 and any(_ends_with(self._tail, p) for p in self.closers):
            self.open_calls -= 1

    @property
    def suppress_eos(self) -> bool:
        """True while a call is open and a closer is known (otherwise EOS is the only way out)."""
        return self.open_calls > 0 and bool(self.closers)
