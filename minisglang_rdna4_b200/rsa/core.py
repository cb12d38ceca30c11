"""Markovian recursive self-aggregation.

Round 0 draws ``n`` independent answers. In each of the next ``t - 1`` rounds every slot draws
``k`` answers of the previous round (its own included) and asks the model to aggregate them into
a better one; only the tail of each candidate (``tail_tokens`` characters' worth) is shown, so
the state carried between rounds is bounded ("Markovian"). The final answer is chosen by
``selection``: ``vote`` (most common normalised final line), ``first`` or ``longest``.

``generate`` is any awaitable ``(messages, max_tokens, temperature, top_p) -> str`` — the
in-process frontend client or an HTTP client.
"""
from __future__ import annotations

import asyncio
import random
import re
from collections import Counter
from dataclasses import dataclass
from typing import Awaitable, Callable, Dict, List, Optional, Sequence

Generate = Callable[[List[Dict[str, str]], int, float, float], Awaitable[str]]


@dataclass(frozen=True)
class RSAParams:
    n: int = 4
    k: int = 2
    t: int = 2
    tail_tokens: int = 1024
    max_tokens: int = 1024
    agg_max_tokens: int = 1024
    temperature: float = 0.7
    top_p: float = 0.95
    selection: str = "vote"
    max_concurrency: int = 8
    max_retries: int = 1
    seed: int = 0

    @staticmethod
    def from_effort(effort: Optional[str]) -> Optional["RSAParams"]:
        """``reasoning_effort`` → ladder (python/minisgl/server/api_server.py:1204)."""
        ladder = {"low": None, "medium": RSAParams(n=2, k=2, t=2), "high": RSAParams(n=4, k=2, t=3),
                  "max": RSAParams(n=8, k=3, t=4)}
        return ladder.get((effort or "").lower())


AGG_TEMPLATE = (
    "You are given a problem and {k} candidate solutions. Some may be wrong. Combine their correct "
    "parts into one improved, complete solution. End with the final answer on its own line.\n\n"
    "Problem:\n{problem}\n\n{candidates}\n\nImproved solution:"
)


def _tail(text: str, limit_chars: int) -> str:
    return text if len(text) <= limit_chars else "…" + text[-limit_chars:]


def _final_line(text: str) -> str:
    lines = [ln.strip() for ln in text.strip().splitlines() if ln.strip()]
    last = lines[-1] if lines else ""
    return re.sub(r"[^0-9a-z.+\-/]", "", last.lower())


def select(answers: Sequence[str], how: str) -> str:
    if not answers:
        return ""
    if how == "first":
        return answers[0]
    if how == "longest":
        return max(answers, key=len)
    votes = Counter(_final_line(a) for a in answers)
    best, _ = votes.most_common(1)[0]
    return next(a for a in answers if _final_line(a) == best)


async def run_rsa(messages: List[Dict[str, str]], params: RSAParams, generate: Generate) -> Dict[str, object]:
    rng = random.Random(params.seed)
    sem = asyncio.Semaphore(params.max_concurrency)
    problem = next((m["content"] for m in reversed(messages) if m.get("role") == "user"), "")
    calls = 0

    async def call(msgs, max_tokens) -> str:
        nonlocal calls
        async with sem:
            for attempt in range(params.max_retries + 1):
                try:
                    calls += 1
                    return await generate(msgs, max_tokens, params.temperature, params.top_p)
                except Exception:
                    if attempt == params.max_retries:
                        return ""
        return ""

    pool = list(await asyncio.gather(*[call(messages, params.max_tokens) for _ in range(params.n)]))
    history = [pool]
    for _ in range(1, params.t):
        jobs = []
        for i in range(params.n):
            others = [j for j in range(params.n) if j != i and pool[j]]
            picks = [i] + rng.sample(others, min(params.k - 1, len(others)))
            cands = "\n\n".join(f"Candidate {c + 1}:\n{_tail(pool[p], params.tail_tokens * 4)}" for c, p in enumerate(picks))
            prompt = AGG_TEMPLATE.format(k=len(picks), problem=problem, candidates=cands)
            jobs.append(call(messages[:-1] + [{"role": "user", "content": prompt}], params.agg_max_tokens))
        new = list(await asyncio.gather(*jobs))
        pool = [n if n else o for n, o in zip(new, pool)]
        history.append(pool)
    return {"answer": select([p for p in pool if p], params.selection), "rounds": len(history), "calls": calls,
            "pool": pool}
