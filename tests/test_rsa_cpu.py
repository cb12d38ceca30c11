import asyncio

from minisglang_rdna4_b200.rsa import RSAParams, run_rsa
from minisglang_rdna4_b200.rsa.core import select


def test_rsa_rounds_calls_and_vote():
    seen = []

    async def gen(msgs, max_tokens, temperature, top_p):
        seen.append(msgs[-1]["content"])
        if "Candidate" in msgs[-1]["content"]:
            return "merged reasoning\nAnswer: 42"
        return f"draft {len(seen)}\nAnswer: {41 + len(seen) % 2}"

    out = asyncio.run(run_rsa([{"role": "user", "content": "6*7?"}], RSAParams(n=4, k=2, t=3), gen))
    assert out["calls"] == 4 * 3 and out["rounds"] == 3
    assert out["answer"].endswith("Answer: 42")
    assert sum("Candidate 2:" in s for s in seen) == 8           # every aggregation saw k = 2 candidates
    assert select(["a\n7", "b\n8", "c\n7"], "vote").endswith("7")
    assert RSAParams.from_effort("high").n == 4 and RSAParams.from_effort("low") is None
