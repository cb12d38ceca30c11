"""Measure-only prefix-reuse oracle (python/minisgl/kvcache/ghost_cache.py:81-215).

It serves nothing. For every admitted prompt it records how many tokens the live prefix cache
reused and how many an ideal cache (no eviction, bounded only by this oracle's own LRU of
chained page hashes) could have reused, because some earlier prompt already covered them. The
difference is what a larger or host-backed KV tier could recover; if it stays a few per cent of
the prompt tokens on real traffic, such a tier has nothing to buy. Off unless
``MSGL_GHOST_ORACLE=1``; cumulative across restarts when ``MSGL_GHOST_ORACLE_DIR`` names a
directory (one JSON file per model and replica, written atomically).

The hash of page p is chained over pages 0..p (FNV-1a 64), so finding it means "an earlier prompt
shared this exact p-page prefix", not "contained this page somewhere".
"""
from __future__ import annotations

import json
import os
from collections import OrderedDict
from typing import Dict, Optional, Sequence

_OFFSET, _PRIME, _MASK = 0xCBF29CE484222325, 0x100000001B3, (1 << 64) - 1


def oracle_enabled() -> bool:
    from ..env import ENV

    return bool(ENV.GHOST_ORACLE.value)


def oracle_path(model: str, dp_rank: int = 0) -> Optional[str]:
    from ..env import ENV

    d = ENV.GHOST_ORACLE_DIR.value
    if not d:
        return None
    slug = "".join(c if c.isalnum() or c in "-._" else "_" for c in (model or "unknown"))
    return os.path.join(d, f"ghost-{slug}-dp{dp_rank}.json")


class GhostPrefixOracle:
    def __init__(self, page_size: int, capacity: int = 1 << 18) -> None:
        self.page_size = max(1, int(page_size))
        self.capacity = int(capacity)
        self._seen: "OrderedDict[int, None]" = OrderedDict()
        self.requests = 0
        self.prompt_tokens = 0
        self.actual_tokens = 0       # reused by the live cache
        self.potential_tokens = 0    # covered by an earlier prompt (upper bound for any tier)

    def _page_hashes(self, tokens: Sequence[int]):
        h = _OFFSET
        ps = self.page_size
        for p in range(len(tokens) // ps):
            for t in tokens[p * ps:(p + 1) * ps]:
                h = ((h ^ (int(t) & _MASK)) * _PRIME) & _MASK
            yield h

    def observe(self, tokens: Sequence[int], cached_len: int) -> int:
        """Account one admitted prompt; returns the tokens an ideal cache would have reused."""
        potential_pages, counting = 0, True
        for h in self._page_hashes(tokens):
            if h in self._seen:
                self._seen.move_to_end(h)
                if counting:
                    potential_pages += 1
            else:
                counting = False          # a prefix match ends at the first unseen page
                self._seen[h] = None
                if len(self._seen) > self.capacity:
                    self._seen.popitem(last=False)
        potential = potential_pages * self.page_size
        self.requests += 1
        self.prompt_tokens += len(tokens)
        self.actual_tokens += int(cached_len)
        # the live cache can never beat the ideal one; keep the bound honest if the oracle's own
        # LRU already forgot a prefix the live cache still holds
        self.potential_tokens += max(potential, int(cached_len))
        return potential

    # ------------------------------------------------------------------ reporting
    def counters(self) -> Dict[str, float]:
        gap = self.potential_tokens - self.actual_tokens
        denom = max(self.prompt_tokens, 1)
        return {"requests": self.requests, "prompt_tokens": self.prompt_tokens, "actual_tokens": self.actual_tokens,
                "potential_tokens": self.potential_tokens, "gap_evict_tokens": gap,
                "actual_share": self.actual_tokens / denom, "gap_evict_share": gap / denom,
                "remembered_pages": len(self._seen)}

    def report(self) -> str:
        c = self.counters()
        return (f"ghost oracle: {c['requests']} prompts, {c['prompt_tokens']} tokens; reused {c['actual_share']:.1%}, "
                f"an unbounded cache would add {c['gap_evict_share']:.1%} "
                f"({c['gap_evict_tokens']} tokens lost to eviction)")

    # ------------------------------------------------------------------ persistence
    def save(self, path: str) -> None:
        tmp = path + ".tmp"
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(tmp, "w") as fh:
            json.dump({"page_size": self.page_size, "capacity": self.capacity, "requests": self.requests,
                       "prompt_tokens": self.prompt_tokens, "actual_tokens": self.actual_tokens,
                       "potential_tokens": self.potential_tokens, "seen": list(self._seen.keys())}, fh)
        os.replace(tmp, path)

    @classmethod
    def load(cls, path: str, page_size: int, capacity: int = 1 << 18) -> "GhostPrefixOracle":
        o = cls(page_size, capacity)
        try:
            with open(path) as fh:
                d = json.load(fh)
        except (OSError, ValueError):
            return o
        if int(d.get("page_size", -1)) != o.page_size:
            return o                      # hashes of another page size are not comparable
        for k in ("requests", "prompt_tokens", "actual_tokens", "potential_tokens"):
            setattr(o, k, int(d.get(k, 0)))
        for h in d.get("seen", [])[-capacity:]:
            o._seen[int(h)] = None
        return o
