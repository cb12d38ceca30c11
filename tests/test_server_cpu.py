"""HTTP contract with a fake backend, message codec, tokenizer worker logic, reasoning and
tool parsing: no GPU, no sockets."""
import asyncio
import json

import pytest
import torch
from fastapi.testclient import TestClient

from minisglang_rdna4_b200.config import ServerArgs
from minisglang_rdna4_b200.core import SamplingParams
from minisglang_rdna4_b200.message import (
    AbortMsg, BatchMsg, DetokenizeMsg, StatsMsg, TokenizeMsg, UserMsg, UserReply, decode_msg, encode_msg,
)
from minisglang_rdna4_b200.server.api_server import FrontendManager, create_app
from minisglang_rdna4_b200.server.args import parse_args
from minisglang_rdna4_b200.server.metrics import FrontendMetrics
from minisglang_rdna4_b200.server.reasoning import ReasoningParser, ReasoningStreamState, derive_delimiters
from minisglang_rdna4_b200.server.tools import ToolCallStreamState, grammar_from_tools, parse_tool_calls
from minisglang_rdna4_b200.tokenizer import ByteTokenizer, DetokenizeManager
from minisglang_rdna4_b200.tokenizer.server import TokenizerWorker


# ------------------------------------------------------------------------------------------ codec
def test_message_codec_round_trip():
    sp = SamplingParams(temperature=0.7, top_k=5, stop=["\n\n"], grammar="json", max_tokens=33)
    msg = BatchMsg(data=[UserMsg(7, torch.arange(5, dtype=torch.int32), sp), AbortMsg(3),
                         DetokenizeMsg(7, 42, True, "stop", logprob=-0.5, top_logprobs=[[42, -0.5], [1, -2.0]])])
    back = decode_msg(encode_msg(msg))
    assert isinstance(back, BatchMsg) and len(back.data) == 3
    assert torch.equal(back.data[0].input_ids, torch.arange(5, dtype=torch.int32))
    assert back.data[0].sampling_params == sp
    assert back.data[2].top_logprobs == [[42, -0.5], [1, -2.0]]
    stats = decode_msg(encode_msg(StatsMsg(1, {"running": 3.0})))
    assert stats.values["running"] == 3.0


# ------------------------------------------------------------------------------------------ detokenizer
def test_detokenizer_stop_strings_and_utf8():
    tok = ByteTokenizer()
    d = DetokenizeManager(tok)
    d.register(1, ["END"], [])
    out = []
    for ch in "hello ENX world END tail".encode():
        text, hit, which = d.step(1, ch, False)
        out.append(text)
        if hit:
            assert which == "END"
            break
    assert "".join(out) == "hello ENX world "
    # stop_keep keeps the matched string
    d.register(2, [], ["</tool_call>"])
    out = []
    for ch in "<tool_call>{}</tool_call>more".encode():
        text, hit, _ = d.step(2, ch, False)
        out.append(text)
        if hit:
            break
    assert "".join(out) == "<tool_call>{}</tool_call>"
    # a multi-byte character is only emitted when complete
    d.register(3, [], [])
    data = "é!".encode()
    t1, _, _ = d.step(3, data[0], False)
    t2, _, _ = d.step(3, data[1], False)
    t3, _, _ = d.step(3, data[2], True)
    assert t1 == "" and t2 == "é" and t3 == "!"


def test_tokenizer_worker_round_trip_and_dp_round_robin():
    args = ServerArgs(model_path="tiny-llama", dp_size=2)
    w = TokenizerWorker(args, ByteTokenizer())
    r0, m0 = w.on_tokenize(TokenizeMsg(1, "abc", SamplingParams(stop=["c"])))
    r1, m1 = w.on_tokenize(TokenizeMsg(2, [{"role": "user", "content": "hi"}], SamplingParams()))
    assert (r0, r1) == (0, 1) and m0.input_ids.tolist() == [97, 98, 99]
    assert "<|im_start|>assistant" in ByteTokenizer().decode(m1.input_ids.tolist())
    reply, abort = w.on_detokenize(DetokenizeMsg(1, ord("a"), False))
    assert reply.incremental_output == "a" and abort is None
    reply, abort = w.on_detokenize(DetokenizeMsg(1, ord("c"), False))
    assert reply.finished and reply.finish_reason == "stop" and abort == 1
    # after a stop hit the request is forgotten: late tokens produce nothing
    assert w.on_detokenize(DetokenizeMsg(1, ord("x"), True)) == (None, None)


# ------------------------------------------------------------------------------------------ reasoning / tools
def test_reasoning_split_streaming_equals_whole():
    p = ReasoningParser("<think>", "</think>")
    text = "<think>step 1\nstep 2</think>\nThe answer is 4."
    assert p.split(text) == ("step 1\nstep 2", "The answer is 4.")
    st = ReasoningStreamState(p)
    r, c = "", ""
    for i in range(0, len(text), 3):
        dr, dc = st.feed(text[i : i + 3])
        r, c = r + dr, c + dc
    dr, dc = st.flush()
    assert (r + dr, c + dc) == ("step 1\nstep 2", "The answer is 4.")
    # generation prompt already opened the span
    p2 = ReasoningParser("<think>", "</think>", starts_open=True)
    assert p2.split("thinking...</think>done") == ("thinking...", "done")
    tmpl = "{% if add_generation_prompt %}<|im_start|>assistant\n<think>\n{% endif %}"
    d = derive_delimiters(tmpl)
    assert d is not None and d.open == "<think>" and d.starts_open
    assert derive_delimiters("plain template") is None


def test_tool_call_parsing_and_forced_grammar():
    text = 'Let me check.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    content, calls = parse_tool_calls(text)
    assert content == "Let me check." and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}
    assert parse_tool_calls("no calls here") == ("no calls here", [])
    st = ToolCallStreamState()
    sent = "".join(st.feed(text[i : i + 5]) for i in range(0, len(text), 5))
    rest, calls2 = st.finish()
    assert sent == "Let me check." and rest == "" and calls2[0]["function"]["name"] == "get_weather"
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}},
             {"type": "function", "function": {"name": "g"}}]
    assert grammar_from_tools(tools, "auto") is None
    schema = json.loads(grammar_from_tools(tools, {"type": "function", "function": {"name": "g"}}))
    assert schema["properties"]["name"]["const"] == "g"
    assert "anyOf" in json.loads(grammar_from_tools(tools, "required"))
    with pytest.raises(ValueError):
        grammar_from_tools(tools, {"function": {"name": "nope"}})


# ------------------------------------------------------------------------------------------ HTTP contract
class FakeManager(FrontendManager):
    """Answers every request with a fixed script of replies."""

    def __init__(self, args, script):
        super().__init__(args)
        self.script = script
        self.sent = []

    async def send_one(self, msg):
        self.sent.append(msg)
        if isinstance(msg, TokenizeMsg):
            for r in self.script(msg):
                self.queues[msg.uid].put_nowait(r)


def _client(script, template=None):
    args = ServerArgs(model_path="tiny-llama", served_model_name="tiny")
    mgr = FakeManager(args, script)
    return TestClient(create_app(args, mgr, template)), mgr


def _words(uid, words, reason="stop", **kw):
    out = []
    for i, w in enumerate(words):
        last = i == len(words) - 1
        out.append(UserReply(uid, w, last, reason if last else None, [i], prompt_tokens=5, cached_tokens=2, **kw))
    return out


def test_models_health_metrics():
    c, mgr = _client(lambda m: _words(m.uid, ["a"]))
    assert c.get("/health").json() == {"status": "ok"}
    assert c.get("/v1/models").json()["data"][0]["id"] == "tiny"
    mgr.metrics.on_scheduler_stats(0, {"running": 2.0, "kv_tokens_used": 64.0})
    body = c.get("/metrics").text
    assert "minisgl_requests_total" in body and 'minisgl_scheduler_running{dp_rank="0"} 2.0' in body
    assert "minisgl_time_to_first_token_seconds_bucket" in body


def test_chat_completion_non_streaming_shape_and_usage():
    c, mgr = _client(lambda m: _words(m.uid, ["Hel", "lo", "!"], "length"))
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                             "temperature": 0.2, "stop": "\n"})
    body = r.json()
    assert r.status_code == 200 and body["object"] == "chat.completion"
    assert body["choices"][0]["message"] == {"role": "assistant", "content": "Hello!"}
    assert body["choices"][0]["finish_reason"] == "length"
    assert body["usage"] == {"prompt_tokens": 5, "completion_tokens": 3, "total_tokens": 8,
                             "prompt_tokens_details": {"cached_tokens": 2}}
    sent = mgr.sent[0]
    assert sent.sampling_params.max_tokens == 3 and sent.sampling_params.stop == ["\n"]
    assert sent.text == [{"role": "user", "content": "hi"}]


def test_chat_completion_streaming_sse_with_reasoning_and_tools():
    tmpl = "<think></think><tool_call></tool_call>"
    words = ["<think>hm", "m</think>", "Sure.", '<tool_call>{"name": "f", "argu', 'ments": {}}</tool_call>']
    c, _ = _client(lambda m: _words(m.uid, words), tmpl)
    tools = [{"type": "function", "function": {"name": "f"}}]
    with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}],
                                                        "stream": True, "tools": tools,
                                                        "stream_options": {"include_usage": True}}) as r:
        chunks = [line[6:] for line in r.iter_lines() if line.startswith("data: ")]
    assert chunks[-1] == "[DONE]"
    objs = [json.loads(x) for x in chunks[:-1]]
    deltas = [o["choices"][0]["delta"] for o in objs if o["choices"]]
    assert "".join(d.get("reasoning_content", "") for d in deltas) == "hmm"
    assert "".join(d.get("content", "") or "" for d in deltas) == "Sure."
    calls = [d["tool_calls"][0] for d in deltas if "tool_calls" in d]
    assert calls and calls[0]["function"]["name"] == "f"
    finals = [o["choices"][0]["finish_reason"] for o in objs if o["choices"] and o["choices"][0]["finish_reason"]]
    assert finals == ["tool_calls"]
    assert objs[-1]["usage"]["completion_tokens"] == len(words)


def test_completions_endpoint_and_validation():
    c, mgr = _client(lambda m: _words(m.uid, ["x", "y"]))
    r = c.post("/v1/completions", json={"prompt": "abc", "max_tokens": 2})
    assert r.json()["choices"][0]["text"] == "xy" and r.json()["object"] == "text_completion"
    assert mgr.sent[0].text == "abc"
    # what the server cannot honour is a 400 with the OpenAI error object, naming the field
    for body, param, code in (
            ({"max_tokens": 2}, "messages", "missing_required_parameter"),          # no prompt / messages
            ({"prompt": "a", "max_tokens": 0}, "max_tokens", "invalid_value"),
            ({"prompt": "a", "n": 2}, "n", "unsupported_parameter"),
            ({"prompt": "a", "logit_bias": {"1": 2}}, "logit_bias", "unsupported_parameter"),
            ({"prompt": "a", "best_of": 3}, "best_of", "unsupported_parameter"),
            ({"prompt": "a", "echo": True}, "echo", "unsupported_parameter"),
            ({"prompt": "a", "suffix": "x"}, "suffix", "unsupported_parameter"),
            ({"prompt": "a", "temperature": "hot"}, "temperature", "invalid_value"),
            ({"messages": [{"role": "user", "content": "hi"}]}, "messages", "unsupported_parameter"),   # raw lane
            ({"prompt": "a", "tools": [{"type": "function", "function": {"name": "f"}}]}, "tools",
             "unsupported_parameter"),
            ({"prompt": "a", "rsa": True}, "rsa", "unsupported_parameter")):
        r = c.post("/v1/completions", json=body)
        assert r.status_code == 400, body
        err = r.json()["error"]
        assert err["type"] == "invalid_request_error" and err["param"] == param and err["code"] == code, (body, err)
        assert err["message"]
    # ignored OpenAI fields are accepted
    assert c.post("/v1/completions", json={"prompt": "a", "user": "u", "store": False}).status_code == 200
    # default max_tokens applies when none is given
    c.post("/v1/completions", json={"prompt": "a"})
    assert mgr.sent[-1].sampling_params.max_tokens == 1024
    # response_format -> grammar
    c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "j"}],
                                         "response_format": {"type": "json_object"}})
    assert mgr.sent[-1].sampling_params.grammar == "json" and mgr.sent[-1].sampling_params.grammar_required


def test_backend_error_becomes_http_400_and_generate_streams():
    c, _ = _client(lambda m: [UserReply(m.uid, "", True, "error", error="prompt too long")])
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 400 and "prompt too long" in r.json()["detail"]
    c2, _ = _client(lambda m: _words(m.uid, ["a", "b"]))
    with c2.stream("POST", "/generate", json={"prompt": "p", "max_tokens": 2}) as r:
        lines = [ln for ln in r.iter_lines() if ln.startswith("data: ")]
    assert lines == ["data: a", "data: b", "data: [DONE]"]


def test_cli_flags_and_aliases():
    a = parse_args(["--model", "m", "--tp-size", "2", "--graph", "64", "--max-running-requests", "128",
                    "--attn", "fi", "--spec-algorithm", "ngram", "--spec-num-draft", "3", "--dummy-weight"])
    assert a.tp_size == 2 and a.cuda_graph_max_bs == 64 and a.max_running_req == 64
    assert a.spec_algorithm == "ngram" and a.spec_num_draft == 3 and a.use_dummy_weight
    with pytest.raises(SystemExit):
        parse_args(["--model", "m", "--enable-ep"])
    assert parse_args(["--model", "m"]).port == 1919


def test_metrics_lifecycle():
    m = FrontendMetrics("x")
    m.on_request(1)
    m.on_token(1)
    m.on_token(1, 3)
    m.on_finish(1, "stop", prompt_tokens=10, cached_tokens=4)
    assert m.counters["generation_tokens_total"] == 4 and m.counters["requests_finished_total"] == 1
    assert m.ttft.n == 1 and m.tpot.n == 1 and m.e2e.n == 1


def test_rsa_requests_run_rollouts_aggregation_rounds_and_a_vote():
    """``rsa`` on a chat request: N rollouts, T - 1 aggregation rounds that each see K candidates, then a
    vote on the final lines. ``reasoning_effort`` alone only does so when the server enabled the ladder."""
    from minisglang_rdna4_b200.server.args import parse_args

    def script(m):
        text = m.text[-1]["content"]
        if "candidate solutions" in text:                    # an aggregation call
            return _words(m.uid, ["merged\n", "42"])
        n = sum(1 for s in mgr.sent if isinstance(s, TokenizeMsg))
        return _words(m.uid, ["guess\n", "42" if n % 3 else "41"])

    c, mgr = _client(script)
    body = {"messages": [{"role": "user", "content": "What is 6 x 7?"}], "rsa": {"n": 3, "k": 2, "t": 2}}
    r = c.post("/v1/chat/completions", json=body)
    out = r.json()
    assert r.status_code == 200 and out["rsa"] == {"rounds": 2, "calls": 6, "n": 3, "k": 2, "t": 2}
    assert out["choices"][0]["message"]["content"].endswith("42") and out["usage"]["completion_tokens"] == 12
    rollouts = [s for s in mgr.sent if isinstance(s, TokenizeMsg)]
    assert len(rollouts) == 6 and all(s.sampling_params.temperature == 0.7 for s in rollouts)
    assert sum("Candidate 2:" in s.text[-1]["content"] for s in rollouts) == 3

    assert c.post("/v1/chat/completions", json={**body, "rsa": {"rounds": 9}}).status_code == 400
    # without the ladder, reasoning_effort is an ordinary request
    c2, mgr2 = _client(lambda m: _words(m.uid, ["x"]))
    c2.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "reasoning_effort": "high"})
    assert len(mgr2.sent) == 1

    args = parse_args(["--model", "tiny-llama", "--rsa-n", "6", "--rsa-selection", "longest", "--rsa-effort-ladder"])
    assert args.rsa.n == 6 and args.rsa.selection == "longest" and args.rsa_effort_ladder
    mgr3 = FakeManager(args, lambda m: _words(m.uid, ["a\n", "7"]))
    c3 = TestClient(create_app(args, mgr3, None))
    out3 = c3.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "q"}],
                                                 "reasoning_effort": "medium", "stream": True})
    assert out3.status_code == 200 and '"rsa"' in out3.text and "[DONE]" in out3.text
    assert sum(isinstance(s, TokenizeMsg) for s in mgr3.sent) == 4     # medium: n = 2, t = 2


def test_reasoning_and_thinking_aliases_fold_into_the_canonical_fields():
    from minisglang_rdna4_b200.server.api_server import OpenAICompletionRequest as Req

    msgs = [{"role": "user", "content": "q"}]
    r = Req(messages=msgs, reasoning={"effort": "high", "max_tokens": 256, "enabled": True})
    assert (r.reasoning_effort, r.reasoning_max_tokens, r.enable_thinking) == ("high", 256, True)
    r = Req(messages=msgs, thinking={"type": "enabled", "budget_tokens": 512})
    assert (r.enable_thinking, r.reasoning_max_tokens) == (True, 512)
    r = Req(messages=msgs, thinking=False, reasoning_max_tokens=64)
    assert r.enable_thinking is False and r.reasoning_max_tokens == 64
    r = Req(messages=msgs, enable_thinking=True, thinking={"type": "disabled"})   # the explicit field wins
    assert r.enable_thinking is True
    with pytest.raises(ValueError):
        Req(messages=msgs, thinking={"type": "sometimes"})
    c, mgr = _client(lambda m: _words(m.uid, ["a"]))
    c.post("/v1/chat/completions", json={"messages": msgs, "thinking": {"type": "disabled"}})
    assert mgr.sent[0].chat_template_kwargs == {"enable_thinking": False}


def test_runaway_tool_call_sent_back_for_continuation_is_refused(monkeypatch):
    """A final assistant turn that ends inside a very large unclosed tool-call block is refused with a
    400 that says why; a short truncated call (the model can still close it) and prose that only
    quotes an opener pass."""
    monkeypatch.setenv("MSGL_TOOLCALL_CONT_LIMIT", "2000")
    c, mgr = _client(lambda m: _words(m.uid, ["ok"]))
    user = {"role": "user", "content": "call it"}
    runaway = "Sure.<tool_call>\n{\"name\": \"write\", \"arguments\": {\"text\": \"" + "a" * 3000
    r = c.post("/v1/chat/completions", json={"messages": [user, {"role": "assistant", "content": runaway}]})
    assert r.status_code == 400
    err = r.json()["error"]
    assert err["code"] == "unclosed_tool_call" and err["param"] == "messages" and "<tool_call>" in err["message"]
    short = "Sure.<tool_call>\n{\"name\": \"write\", \"arguments\": {\"text\": \"abc"
    assert c.post("/v1/chat/completions",
                  json={"messages": [user, {"role": "assistant", "content": short}]}).status_code == 200
    closed = "<tool_call>\n{\"name\": \"write\", \"arguments\": {}}\n</tool_call>" + "b" * 3000
    assert c.post("/v1/chat/completions",
                  json={"messages": [user, {"role": "assistant", "content": closed}]}).status_code == 200
    monkeypatch.setenv("MSGL_TOOLCALL_CONT_LIMIT", "0")
    assert c.post("/v1/chat/completions",
                  json={"messages": [user, {"role": "assistant", "content": runaway}]}).status_code == 200
