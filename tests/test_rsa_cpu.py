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


def test_proxy_fans_out_against_an_upstream_and_forwards_plain_requests():
    import asyncio

    from minisglang_rdna4_b200.rsa import RSAParams
    from minisglang_rdna4_b200.rsa.proxy import handle_chat, params_for

    calls = []

    async def post(path, payload):
        calls.append(payload)
        text = payload["messages"][-1]["content"]
        answer = "merged\n9" if "candidate solutions" in text else f"try {len(calls)}\n9"
        return {"choices": [{"message": {"role": "assistant", "content": answer}}],
                "usage": {"prompt_tokens": 10, "completion_tokens": 4}}

    defaults = RSAParams(n=3, k=2, t=2)
    body = {"model": "m", "messages": [{"role": "user", "content": "3 x 3?"}], "rsa": True, "seed": 1}
    out = asyncio.run(handle_chat(body, post, defaults))
    assert out["rsa"] == {"rounds": 2, "calls": 6, "n": 3, "k": 2, "t": 2} and len(calls) == 6
    assert out["choices"][0]["message"]["content"].endswith("9") and out["usage"]["total_tokens"] == 6 * 14
    assert all(c["stream"] is False and c["model"] == "m" and c["seed"] == 1 for c in calls)

    calls.clear()
    plain = {"messages": [{"role": "user", "content": "hi"}], "reasoning_effort": "high"}
    asyncio.run(handle_chat(plain, post, defaults))
    assert calls == [plain]                                                  # forwarded untouched
    assert params_for(plain, defaults, effort_ladder=True).n == 4            # the ladder, when enabled
    import pytest

    with pytest.raises(ValueError):
        params_for({"rsa": {"rounds": 2}}, defaults, False)
