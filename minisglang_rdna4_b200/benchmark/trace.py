"""Trace replay for the load client (python/minisgl/benchmark/client.py:287-500): requests are
issued at the arrival times recorded in a production trace instead of at a fixed concurrency.

Two JSON-lines formats are read:

* Qwen chat trace: ``chat_id, parent_chat_id, timestamp`` (seconds), ``input_length,
  output_length, type, turn, hash_ids``;
* Mooncake trace: ``timestamp`` (milliseconds), ``input_length, output_length, hash_ids``.

``hash_ids`` name the prompt's blocks of ``block_tokens`` tokens; two requests that share leading
hash ids share that much prompt. The reference ignores them and sends unrelated text; here every
hash id expands to its own deterministic block of words, so a replay exercises the prefix cache
the way the recorded traffic did.

``python -m minisglang_rdna4_b200.benchmark.trace --trace mooncake.jsonl --url http://127.0.0.1:1919
--scale 0.5 --limit 500``
"""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import time
from dataclasses import dataclass, field
from typing import List, Optional

from .client import RequestStat, one_request, percentile


@dataclass
class TraceEntry:
    timestamp: float                 # seconds from the start of the trace
    input_length: int                # tokens
    output_length: int               # tokens
    hash_ids: List[int] = field(default_factory=list)
    chat_id: Optional[int] = None
    parent_chat_id: Optional[int] = None


def read_trace(path: str, fmt: str = "auto", limit: Optional[int] = None) -> List[TraceEntry]:
    out: List[TraceEntry] = []
    with open(path) as fh:
        for line in fh:
            line = line.strip()
            if not line:
                continue
            d = json.loads(line)
            kind = fmt
            if kind == "auto":
                kind = "qwen" if "chat_id" in d else "mooncake"
            ts = float(d["timestamp"]) / (1000.0 if kind == "mooncake" else 1.0)
            out.append(TraceEntry(ts, int(d["input_length"]), int(d["output_length"]),
                                  [int(h) for h in d.get("hash_ids", [])], d.get("chat_id"), d.get("parent_chat_id")))
            if limit is not None and len(out) >= limit:
                break
    return out


def scale_trace(entries: List[TraceEntry], scale: float) -> List[TraceEntry]:
    """Shift the first arrival to 0 and multiply the gaps by ``scale`` (< 1 = faster replay)."""
    if not entries:
        return []
    t0 = min(e.timestamp for e in entries)
    scaled = [TraceEntry((e.timestamp - t0) * scale, e.input_length, e.output_length, e.hash_ids, e.chat_id,
                         e.parent_chat_id) for e in entries]
    return sorted(scaled, key=lambda e: e.timestamp)


def prompt_for(entry: TraceEntry, uid: int, block_tokens: int = 512, words_per_token: float = 1.0) -> str:
    """Deterministic text of about ``input_length`` tokens. Block i is a function of ``hash_ids[i]``
    alone; what the hash ids do not cover is filled with words unique to the request."""
    per_block = max(1, int(block_tokens * words_per_token))
    want = max(1, int(entry.input_length * words_per_token))
    words: List[str] = []
    for h in entry.hash_ids:
        if len(words) >= want:
            break
        rng = random.Random(h)
        words.extend(f"w{rng.randrange(50000)}" for _ in range(min(per_block, want - len(words))))
    if len(words) < want:
        rng = random.Random((uid << 20) ^ 0x5BD1E995)
        words.extend(f"u{rng.randrange(50000)}" for _ in range(want - len(words)))
    return " ".join(words)


def shared_prefix_blocks(a: TraceEntry, b: TraceEntry) -> int:
    n = 0
    for x, y in zip(a.hash_ids, b.hash_ids):
        if x != y:
            break
        n += 1
    return n


async def replay(url: str, model: str, entries: List[TraceEntry], block_tokens: int = 512,
                 words_per_token: float = 1.0, temperature: float = 0.0, max_inflight: int = 1024,
                 request_fn=one_request, sleep=asyncio.sleep, clock=time.perf_counter) -> dict:
    """Issue every entry at its timestamp (late when ``max_inflight`` requests are outstanding)."""
    sem = asyncio.Semaphore(max_inflight)
    stats: List[RequestStat] = []
    lateness: List[float] = []

    async def run(session) -> None:
        start = clock()

        async def timed(i: int, e: TraceEntry) -> RequestStat:
            delay = e.timestamp - (clock() - start)
            if delay > 0:
                await sleep(delay)
            async with sem:
                lateness.append(max(0.0, (clock() - start) - e.timestamp))
                return await request_fn(session, url, model, prompt_for(e, i, block_tokens, words_per_token),
                                        e.output_length, temperature)

        stats.extend(await asyncio.gather(*[timed(i, e) for i, e in enumerate(entries)]))

    t0 = clock()
    if request_fn is one_request:
        import aiohttp

        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None)) as session:
            await run(session)
    else:
        await run(None)
    wall = clock() - t0
    ok = [s for s in stats if s.error is None]
    ttft = [s.ttft for s in ok if s.ttft is not None]
    tpot = [s.tpot for s in ok if s.tpot is not None]
    return {
        "requests": len(entries), "failed": len(stats) - len(ok), "wall_s": wall,
        "trace_span_s": entries[-1].timestamp if entries else 0.0,
        "input_tokens": sum(e.input_length for e in entries),
        "output_tok_s": sum(s.completion_tokens for s in ok) / wall if wall > 0 else 0.0,
        "ttft_p50_ms": 1e3 * percentile(ttft, 0.5), "ttft_p99_ms": 1e3 * percentile(ttft, 0.99),
        "tpot_p50_ms": 1e3 * percentile(tpot, 0.5), "tpot_p99_ms": 1e3 * percentile(tpot, 0.99),
        "issue_lateness_p99_ms": 1e3 * percentile(lateness, 0.99),
        "errors": sorted({s.error for s in stats if s.error})[:3],
    }


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--trace", required=True)
    ap.add_argument("--format", default="auto", choices=["auto", "qwen", "mooncake"])
    ap.add_argument("--url", default="http://127.0.0.1:1919")
    ap.add_argument("--model", default="model")
    ap.add_argument("--scale", type=float, default=1.0, help="multiply inter-arrival gaps (0.5 = twice the rate)")
    ap.add_argument("--limit", type=int, default=None)
    ap.add_argument("--block-tokens", type=int, default=512, help="tokens covered by one hash id")
    ap.add_argument("--words-per-token", type=float, default=1.0)
    ap.add_argument("--max-inflight", type=int, default=1024)
    a = ap.parse_args(argv)
    entries = scale_trace(read_trace(a.trace, a.format, a.limit), a.scale)
    print(json.dumps(asyncio.run(replay(a.url, a.model, entries, a.block_tokens, a.words_per_token,
                                        max_inflight=a.max_inflight))))


if __name__ == "__main__":
    main()
