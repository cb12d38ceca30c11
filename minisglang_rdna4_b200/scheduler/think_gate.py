"""Token-sequence gates (python/minisgl/scheduler/think_gate.py:123 ToolCallGate, :252
ThinkGate).

``ThinkGate`` answers one question per request, on token ids only: has the request left its
reasoning span yet? While the span is open the request's grammar is held back; the span ends when

* the close delimiter has been emitted (a token *sequence*, matched on a rolling window so that
  self-overlapping delimiters are not missed),
* a wildcard closer matched: ``(head, tail, max_gap)`` = ``head``, then at most ``max_gap``
  arbitrary tokens, then ``tail`` (channel-routed templates name the recipient inside the closer),
* the model answered directly without opening a span (an answer-header pattern), or
* a tool call was opened.

A budget forces the close delimiter out token by token when the model keeps thinking past it, and
a verbatim-loop detector spends the budget early when the model re-emits one block over and over
(a looping model puts ~1.0 on the continuation, so nothing but the forced close ends the span).

``observe`` / ``commit_many`` are the only mutators. ``forced_token``, ``forced_at`` and ``scan``
are pure queries: speculative decoding may ask where a candidate chain would release without
advancing the gate, and then commits the accepted tokens once.

``ToolCallGate`` suppresses the end-of-sequence token while a tool call that the model opened has
not been closed, up to a runaway limit after which the request is ended.

No torch, tokenizer or environment access here: the module speaks ``int`` only.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple

Ids = Tuple[int, ...]
Pattern = Tuple[Ids, Ids, int]          # (head, tail, max_gap); empty tail = "window ends with head"


def as_pattern(p) -> Optional[Pattern]:
    """A list of ids, or ``(head, tail, max_gap)``, as a pattern; ``None`` when it is empty."""
    if p is None:
        return None
    if isinstance(p, tuple) and len(p) == 3 and isinstance(p[2], int) and not isinstance(p[0], int):
        head, tail, gap = tuple(int(t) for t in p[0]), tuple(int(t) for t in p[1]), max(int(p[2]), 0)
        if not head and tail:
            head, tail, gap = tail, (), 0
        return (head, tail, gap) if head else None
    ids = tuple(int(t) for t in p)
    return (ids, (), 0) if ids else None


def pattern_width(p: Pattern) -> int:
    return len(p[0]) + (p[2] + len(p[1]) if p[1] else 0)


def _suffix_eq(window: Sequence[int], seq: Ids, end: int) -> bool:
    """Does ``window`` hold ``seq`` ending ``end`` tokens before its right edge?"""
    n = len(seq)
    stop = len(window) - end
    return n > 0 and stop - n >= 0 and tuple(window[stop - n:stop]) == seq


def pattern_matches(window: Sequence[int], pat: Pattern) -> bool:
    head, tail, gap = pat
    if not tail:
        return _suffix_eq(window, head, 0)
    if not _suffix_eq(window, tail, 0):
        return False
    return any(_suffix_eq(window, head, len(tail) + g) for g in range(gap + 1))


def _ends_with(history: Sequence[int], pattern: Sequence[int]) -> bool:
    return _suffix_eq(history, tuple(pattern), 0)


class ThinkGate:
    """See the module docstring. ``close_ids`` is the literal close delimiter (also what the budget
    forces out); ``release_patterns`` are tool-call openers; ``answer_patterns`` are answer-turn
    headers; ``close_wildcards`` are additional ``(head, tail, max_gap)`` closers."""

    def __init__(self, close_ids: Sequence[int], release_patterns: Iterable = (), budget: int = 0,
                 span_open: bool = True, answer_patterns: Iterable = (), close_wildcards: Iterable = (),
                 loop_period: int = 64, loop_span: int = 48, loop_reps: int = 3) -> None:
        self.close_ids: List[int] = [int(t) for t in close_ids]
        pats = [as_pattern(self.close_ids)]
        pats += [as_pattern(p) for p in release_patterns]
        pats += [as_pattern(p) for p in answer_patterns]
        pats += [as_pattern(p) for p in close_wildcards]
        self.patterns: Tuple[Pattern, ...] = tuple(p for p in pats if p is not None)
        self.release_patterns = [list(p) for p in release_patterns]
        self.budget = int(budget)
        self.span_open = bool(span_open)
        self.released = not self.span_open
        self.thought = 0
        self.loop = 0                      # period of a detected verbatim loop (0 = none)
        self._loop_reported = False
        self._forcing = 0                  # index of the next forced close token
        self._width = max([pattern_width(p) for p in self.patterns] + [1])
        self._tail: List[int] = []
        self._loop_period, self._loop_span, self._loop_reps = int(loop_period), int(loop_span), int(loop_reps)
        self._hist: List[int] = []
        self._runs: List[int] = [0] * (self._loop_period + 1)

    # ---- queries (pure) ----
    @property
    def grammar_active(self) -> bool:
        return self.released

    def _over_budget(self, thought: int) -> bool:
        return self.budget > 0 and thought >= self.budget

    def forced_token(self) -> Optional[int]:
        """Token the sampler must emit next (budget exhausted or loop detected), or None."""
        return self.forced_at(0)

    def forced_at(self, ahead: int) -> Optional[int]:
        """Forced token ``ahead`` positions from now, assuming every position up to it emits what
        the gate forces (verify rows of a speculative step ask this for the rows after the first)."""
        if self.released or not self.close_ids:
            return None
        if self._forcing > 0:
            i = self._forcing + ahead
            return self.close_ids[i] if i < len(self.close_ids) else None
        if self.budget <= 0:
            return None
        start = max(self.budget - self.thought, 0)      # positions until the budget is reached
        if ahead < start:
            return None
        i = ahead - start
        return self.close_ids[i] if i < len(self.close_ids) else None

    def scan(self, tokens: Sequence[int]) -> Optional[int]:
        """Index in ``tokens`` at which a chain of candidate tokens would release the gate (the
        gate's state is not touched), or None when it would not."""
        if self.released:
            return None
        window = list(self._tail)
        for i, tok in enumerate(tokens):
            window.append(int(tok))
            if len(window) > self._width:
                del window[: len(window) - self._width]
            if any(pattern_matches(window, p) for p in self.patterns):
                return i
        return None

    def take_loop_report(self) -> int:
        """Period of a loop detected since the last call, or 0 (reported once; for the log)."""
        if not self.loop or self._loop_reported:
            return 0
        self._loop_reported = True
        return self.loop

    # ---- mutators ----
    def observe(self, token: int) -> bool:
        """Commit one emitted token. Returns True when this token released the gate."""
        if self.released:
            return False
        token = int(token)
        self.thought += 1
        self._tail.append(token)
        if len(self._tail) > self._width:
            del self._tail[: len(self._tail) - self._width]
        if self._forcing > 0 or self._over_budget(self.thought - 1):
            if self._forcing < len(self.close_ids) and token == self.close_ids[self._forcing]:
                self._forcing += 1
                if self._forcing == len(self.close_ids):
                    self.released = True
                return self.released
            self._forcing = 0                            # a free-running sampler ignored the force
        if any(pattern_matches(self._tail, p) for p in self.patterns):
            self.released = True
            return True
        self._loop_step(token)
        return False

    def commit_many(self, tokens: Sequence[int]) -> Optional[int]:
        """Commit accepted tokens in order; index of the releasing token, or None."""
        for i, t in enumerate(tokens):
            if self.observe(t):
                return i
        return None

    def _loop_step(self, token: int) -> None:
        """``runs[p]`` counts consecutive tokens equal to the token ``p`` back: a unit of ``p`` tokens
        repeated ``r`` times gives ``runs[p] == p * (r - 1)``. A run of at least ``loop_span`` tokens
        that covers ``loop_reps`` repeats spends the budget; the floors keep tables, rulers and
        short lists from triggering it."""
        hist, runs = self._hist, self._runs
        n = len(hist)
        for p in range(1, min(self._loop_period, n) + 1):
            if hist[n - p] == token:
                runs[p] += 1
                if not self.loop and runs[p] >= self._loop_span and runs[p] >= p * self._loop_reps:
                    self.loop = p
                    if self.close_ids:
                        self.budget = min(self.budget, self.thought) if self.budget > 0 else self.thought
            else:
                runs[p] = 0
        hist.append(token)
        if len(hist) > self._loop_period:
            del hist[0]


class ToolCallGate:
    """Follows tool-call openers and closers on token ids. ``limit`` bounds the tokens one open
    call may run for: past it the call is a runaway (a degenerate model can loop inside a call
    forever because EOS is masked there) and the scheduler ends the request."""

    def __init__(self, openers: Sequence[Sequence[int]], closers: Sequence[Sequence[int]], limit: int = 8192) -> None:
        self.openers = [list(map(int, p)) for p in openers if len(p)]
        self.closers = [list(map(int, p)) for p in closers if len(p)]
        self.limit = int(limit)
        self.open_calls = 0
        self.calls_seen = 0
        self.inside = 0                                   # tokens since the current call opened
        self.runaway = False
        self._tail: List[int] = []
        self._keep = max([len(p) for p in self.openers + self.closers] + [1])

    def observe(self, token: int) -> None:
        self._tail.append(int(token))
        if len(self._tail) > self._keep:
            del self._tail[: len(self._tail) - self._keep]
        if any(_ends_with(self._tail, p) for p in self.openers):
            self.open_calls += 1
            self.calls_seen += 1
            self.inside = 0
        elif self.open_calls > 0 and any(_ends_with(self._tail, p) for p in self.closers):
            self.open_calls -= 1
            self.inside = 0
        elif self.open_calls > 0:
            self.inside += 1
            if self.limit > 0 and self.inside >= self.limit:
                self.runaway = True

    @property
    def is_open(self) -> bool:
        return self.open_calls > 0

    @property
    def suppress_eos(self) -> bool:
        """True while a call is open and a closer is known (otherwise EOS is the only way out)."""
        return self.open_calls > 0 and bool(self.closers) and not self.runaway
