"""Asynchronous load client for the OpenAI-compatible server (python/minisgl/benchmark/client.py,
methodology of tools/serve_perf.py:7-23): drives ``concurrency`` streaming requests at a time with
distinct prompt suffixes (so the prefix cache cannot make later requests free), discards the
warm-up requests, and reports true output tok/s = sum(usage.completion_tokens) / wall time plus
TTFT / TPOT percentiles.

``python -m minisglang_rdna4_b200.benchmark.client --url http://127.0.0.1:1919 --requests 64
--concurrency 16 --prompt-tokens 512 --max-tokens 128``
"""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import time
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class RequestStat:
    ttft: Optional[float] = None
    latency: float = 0.0
    completion_tokens: int = 0
    chunks: int = 0
    error: Optional[str] = None

    @property
    def tpot(self) -> Optional[float]:
        if self.ttft is None or self.completion_tokens < 2:
            return None
        return (self.latency - self.ttft) / (self.completion_tokens - 1)


def percentile(xs: List[float], q: float) -> float:
    if not xs:
        return float("nan")
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))]


def make_prompt(n_words: int, rng: random.Random, uid: int) -> str:
    words = [f"w{rng.randrange(50000)}" for _ in range(n_words)]
    return f"request {uid}: " + " ".join(words)


async def one_request(session, url: str, model: str, prompt: str, max_tokens: int, temperature: float) -> RequestStat:
    stat = RequestStat()
    body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens,
            "temperature": temperature, "stream": True, "stream_options": {"include_usage": True},
            "ignore_eos": True}
    t0 = time.perf_counter()
    try:
        async with session.post(url + "/v1/chat/completions", json=body) as resp:
            if resp.status != 200:
                stat.error = f"HTTP {resp.status}: {(await resp.text())[:200]}"
                return stat
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data: "):
                    continue
                data = line[6:]
                if data == "[DONE]":
                    break
                obj = json.loads(data)
                if obj.get("usage"):
                    stat.completion_tokens = obj["usage"]["completion_tokens"]
                for choice in obj.get("choices", []):
                    delta = choice.get("delta", {})
                    if delta.get("content") or delta.get("reasoning_content"):
                        stat.chunks += 1
                        if stat.ttft is None:
                            stat.ttft = time.perf_counter() - t0
    except Exception as exc:  # connection errors count as failed requests
        stat.error = repr(exc)
    stat.latency = time.perf_counter() - t0
    if stat.completion_tokens == 0:
        stat.completion_tokens = stat.chunks
    return stat


async def run_load(url: str, model: str, requests: int, concurrency: int, prompt_words: int, max_tokens: int,
                   temperature: float = 0.0, warmup: int = 0, seed: int = 0) -> dict:
    import aiohttp

    rng = random.Random(seed)
    sem = asyncio.Semaphore(concurrency)
    stats: List[RequestStat] = []

    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None)) as session:
        async def guarded(i: int) -> RequestStat:
            async with sem:
                return await one_request(session, url, model, make_prompt(prompt_words, rng, i), max_tokens, temperature)

        if warmup:
            await asyncio.gather(*[guarded(-1 - i) for i in range(warmup)])
        t0 = time.perf_counter()
        stats = await asyncio.gather(*[guarded(i) for i in range(requests)])
        wall = time.perf_counter() - t0
    ok = [s for s in stats if s.error is None]
    ttft = [s.ttft for s in ok if s.ttft is not None]
    tpot = [s.tpot for s in ok if s.tpot is not None]
    return {
        "requests": requests, "failed": len(stats) - len(ok), "wall_s": wall,
        "output_tok_s": sum(s.completion_tokens for s in ok) / wall if wall > 0 else 0.0,
        "ttft_p50_ms": 1e3 * percentile(ttft, 0.5), "ttft_p99_ms": 1e3 * percentile(ttft, 0.99),
        "tpot_p50_ms": 1e3 * percentile(tpot, 0.5), "tpot_p99_ms": 1e3 * percentile(tpot, 0.99),
        "latency_p50_s": percentile([s.latency for s in ok], 0.5),
        "errors": sorted({s.error for s in stats if s.error})[:3],
    }


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:1919")
    ap.add_argument("--model", default="model")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--concurrency", type=int, default=16)
    ap.add_argument("--prompt-tokens", type=int, default=512, help="approximate prompt length in words")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args(argv)
    out = asyncio.run(run_load(a.url, a.model, a.requests, a.concurrency, a.prompt_tokens, a.max_tokens,
                               a.temperature, a.warmup))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
