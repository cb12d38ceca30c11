import asyncio
import json

from minisglang_rdna4_b200.benchmark.client import RequestStat
from minisglang_rdna4_b200.benchmark.trace import (prompt_for, read_trace, replay, scale_trace,
                                                   shared_prefix_blocks)


def _write(path, rows):
    with open(path, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")


def test_read_scale_and_prefix_sharing(tmp_path):
    moon = str(tmp_path / "moon.jsonl")
    _write(moon, [
        {"timestamp": 3000, "input_length": 1100, "output_length": 20, "hash_ids": [7, 8, 9]},
        {"timestamp": 1000, "input_length": 1030, "output_length": 10, "hash_ids": [7, 8, 11]},
    ])
    qwen = str(tmp_path / "qwen.jsonl")
    _write(qwen, [{"chat_id": 5, "parent_chat_id": -1, "timestamp": 12.5, "input_length": 40, "output_length": 7,
                   "type": "text", "turn": 1, "hash_ids": [1]}])
    m = read_trace(moon)
    assert [e.timestamp for e in m] == [3.0, 1.0] and m[0].hash_ids == [7, 8, 9]
    q = read_trace(qwen)
    assert q[0].timestamp == 12.5 and q[0].chat_id == 5 and read_trace(moon, limit=1)[0].input_length == 1100
    s = scale_trace(m, 0.5)
    assert [e.timestamp for e in s] == [0.0, 1.0] and s[0].input_length == 1030      # sorted, first arrival at 0

    a, b = prompt_for(m[0], 0).split(), prompt_for(m[1], 1).split()
    assert len(a) == 1100 and len(b) == 1030
    assert shared_prefix_blocks(m[0], m[1]) == 2 and a[:1024] == b[:1024] and a[1024] != b[1024]
    assert prompt_for(q[0], 3) == prompt_for(q[0], 3) and len(prompt_for(q[0], 3).split()) == 40


def test_replay_issues_requests_at_their_timestamps():
    now = [0.0]
    issued = []

    async def fake_sleep(dt):
        now[0] += dt

    async def fake_request(session, url, model, prompt, max_tokens, temperature):
        issued.append((round(now[0], 3), len(prompt.split()), max_tokens))
        st = RequestStat(ttft=0.01, latency=0.01 + 0.002 * (max_tokens - 1), completion_tokens=max_tokens)
        return st

    from minisglang_rdna4_b200.benchmark.trace import TraceEntry

    entries = [TraceEntry(0.0, 30, 4, [1]), TraceEntry(0.5, 50, 8, [1, 2]), TraceEntry(2.0, 10, 2)]
    out = asyncio.run(replay("http://x", "m", entries, block_tokens=16, request_fn=fake_request, sleep=fake_sleep,
                             clock=lambda: now[0]))
    assert sorted(issued) == [(0.0, 30, 4), (0.5, 50, 8), (2.0, 10, 2)]
    assert out["requests"] == 3 and out["failed"] == 0 and out["input_tokens"] == 90
    assert abs(out["tpot_p50_ms"] - 2.0) < 1e-6 and out["trace_span_s"] == 2.0
