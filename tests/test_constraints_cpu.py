"""Structured output and gates on the CPU engine with the byte tokenizer: a JSON grammar must
yield parseable JSON from a random-weight model; a reasoning budget forces the close
delimiter; an open tool call suppresses end-of-sequence."""
import json

import torch

from minisglang_rdna4_b200 import SamplingParams
from minisglang_rdna4_b200.llm import LLM
from minisglang_rdna4_b200.models.config import ModelConfig, RotaryConfig
from minisglang_rdna4_b200.scheduler.think_gate import ThinkGate, ToolCallGate
from minisglang_rdna4_b200.tokenizer import ByteTokenizer


def _cfg():
    return ModelConfig(num_layers=1, num_qo_heads=2, num_kv_heads=1, head_dim=32, hidden_size=64, vocab_size=260,
                       intermediate_size=128, rms_norm_eps=1e-6,
                       rotary_config=RotaryConfig(32, 32, 512, 1e4), model_type="llama", torch_dtype="float32",
                       max_position_embeddings=512, eos_token_ids=(257,))


def _llm():
    return LLM(model_config=_cfg(), use_dummy_weight=True, device="cpu", page_size=16, max_running_req=4,
               num_page_override=64, seed=3)


def test_json_schema_grammar_produces_valid_json():
    llm = _llm()
    schema = json.dumps({"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "boolean"}},
                         "required": ["a", "b"], "additionalProperties": False})
    prompt = list(b"give me json:")
    outs = llm.generate([prompt, prompt], [SamplingParams(max_tokens=60, grammar=schema, temperature=0.8, top_k=40),
                                           SamplingParams(max_tokens=8, ignore_eos=True)])
    text = ByteTokenizer().decode(outs[0].token_ids)
    obj = json.loads(text)
    assert set(obj) == {"a", "b"} and isinstance(obj["a"], int) and isinstance(obj["b"], bool)
    assert outs[0].finish_reason == "stop"          # the grammar terminated and only EOS was left
    assert len(outs[1].token_ids) == 8              # the unconstrained neighbour is untouched


def test_think_gate_budget_and_release():
    g = ThinkGate(close_ids=[5, 6], budget=3)
    for t in (1, 2, 3):
        assert g.forced_token() is None
        g.observe(t)
    assert g.forced_token() == 5
    g.observe(5)
    assert g.forced_token() == 6 and not g.released
    g.observe(6)
    assert g.released and g.forced_token() is None
    g2 = ThinkGate(close_ids=[9, 9], release_patterns=[[7, 8]])
    g2.observe(7)
    assert not g2.grammar_active
    g2.observe(8)
    assert g2.grammar_active            # a tool-call opener ends the span too
    assert ThinkGate(close_ids=[1], span_open=False).grammar_active


def test_think_gate_sequences_wildcards_and_direct_answers():
    # a self-overlapping close delimiter: a cursor that resets on divergence would miss (4, 4, 5) in 4 4 4 5
    g = ThinkGate(close_ids=[4, 4, 5])
    for t in (4, 4, 4):
        g.observe(t)
        assert not g.released
    assert g.observe(5) and g.released
    # delimiters that share their last token: the opener 328 19669 200023 must not release the gate
    close = [200007, 200022, 140680, 328, 76976, 200023]
    g = ThinkGate(close_ids=close, answer_patterns=[[328, 76976, 200023]])
    assert g.commit_many([328, 19669, 200023, 11, 12]) is None and not g.released
    assert g.commit_many(close) == len(close) - 1
    # ... and answering directly (the answer-turn header without a reasoning turn) releases it as well
    g = ThinkGate(close_ids=close, answer_patterns=[[328, 76976, 200023]])
    assert g.commit_many([7, 328, 76976, 200023]) == 3
    # wildcard closer: head, at most two arbitrary tokens (the recipient), tail
    g = ThinkGate(close_ids=[1, 2, 3], close_wildcards=[((50, 51), (60,), 2)])
    assert g.scan([9, 50, 51, 7, 8, 60]) == 5              # pure query: nothing advanced
    assert not g.released and g.thought == 0
    assert g.commit_many([9, 50, 51, 7, 8, 9, 60]) is None  # three tokens in between: no match
    assert g.commit_many([50, 51, 60]) == 2
    # what a speculative verify row k tokens ahead would be forced to
    g = ThinkGate(close_ids=[5, 6], budget=3)
    g.observe(1)
    assert [g.forced_at(a) for a in range(5)] == [None, None, 5, 6, None]


def test_think_gate_loop_detector_spends_the_budget():
    g = ThinkGate(close_ids=[99], budget=10_000, loop_period=16, loop_span=24, loop_reps=3)
    block = [11, 12, 13, 14, 15, 16]
    n = 0
    for t in [1, 2, 3] + block * 10:
        if g.forced_token() is not None:
            break
        g.observe(t)
        n += 1
    assert g.loop == len(block) and g.take_loop_report() == len(block) and g.take_loop_report() == 0
    assert n < 3 + len(block) * 6                      # caught within a few repeats, far below the budget
    assert g.forced_token() == 99
    g.observe(99)
    assert g.released
    # legitimate short repetition (a ruler, a short list) stays below the span floor
    g = ThinkGate(close_ids=[99], budget=0, loop_period=16, loop_span=24, loop_reps=3)
    for t in [7] * 20 + list(range(100, 140)) + [8, 9] * 8:
        g.observe(t)
    assert g.loop == 0 and g.forced_token() is None
    # without a budget the detector still closes an endless loop
    g = ThinkGate(close_ids=[99], budget=0, loop_period=16, loop_span=24, loop_reps=3)
    for t in block * 8:
        g.observe(t)
    assert g.forced_token() == 99


def test_tool_call_gate_runaway_limit():
    g = ToolCallGate(openers=[[10]], closers=[[12]], limit=5)
    g.observe(10)
    for _ in range(4):
        g.observe(3)
    assert g.suppress_eos and not g.runaway
    g.observe(3)
    assert g.runaway and not g.suppress_eos


def test_tool_call_gate_suppresses_eos_until_closed():
    g = ToolCallGate(openers=[[10, 11]], closers=[[12]])
    assert not g.suppress_eos
    g.observe(10)
    g.observe(11)
    assert g.suppress_eos
    g.observe(3)
    g.observe(12)
    assert not g.suppress_eos


def test_reasoning_budget_forces_close_delimiter_end_to_end():
    llm = _llm()
    sp = SamplingParams(max_tokens=12, ignore_eos=True, think_close_delim="</t>", think_budget=4, think_span_open=True)
    out = llm.generate([list(b"hello")], sp)[0]
    text = ByteTokenizer().decode(out.token_ids)
    assert text[4:8] == "</t>", text


def test_end_of_turn_is_suppressed_inside_a_budgeted_reasoning_span():
    """A thinking model must not end its turn in the middle of a reasoning span: while the span the
    prompt opened is still open (and a budget will close it), the end-of-sequence ids are masked."""
    prompt = [list(b"hello")]
    plain = _llm().generate(prompt, SamplingParams(max_tokens=4, ignore_eos=True))[0].token_ids
    stop = plain[0]                                   # what the model wants to say first

    llm = _llm()
    llm.eos_ids = {stop}                              # pretend that token ends the turn
    free = llm.generate(prompt, SamplingParams(max_tokens=8))[0]
    assert free.token_ids == [stop]                   # without a gate the turn ends at once

    llm = _llm()
    llm.eos_ids = {stop}
    sp = SamplingParams(max_tokens=8, think_close_delim="</t>", think_budget=3, think_span_open=True)
    gated = llm.generate(prompt, sp)[0].token_ids
    text = ByteTokenizer().decode(gated)
    assert stop not in gated[:3] and "</t>" in text   # three thought tokens, then the forced close
