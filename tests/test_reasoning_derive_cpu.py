"""Reasoning delimiters derived from a tokenizer's own chat template (reference behaviour:
python/minisgl/server/reasoning.py:654-912)."""
import pytest

from minisglang_rdna4_b200.server.reasoning import (derive_from_history, derive_from_thinking_switch,
                                                    derive_from_tokenizer, resolve_reasoning_parser)


def _tok(template, specials):
    tokenizers = pytest.importorskip("tokenizers")
    from transformers import PreTrainedTokenizerFast

    vocab = {"<unk>": 0, "hi": 1}
    t = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="<unk>"))
    t.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok = PreTrainedTokenizerFast(tokenizer_object=t, unk_token="<unk>")
    tok.add_special_tokens({"additional_special_tokens": list(specials)})
    tok.chat_template = template
    return tok


_HEAD = ("{% for m in messages %}<|im_start|>{{ m.role }}\n"
         "{% if m.reasoning_content %}<think>\n{{ m.reasoning_content }}\n</think>\n\n{% endif %}"
         "{{ m.content }}<|im_end|>\n{% endfor %}")
_SPECIALS = ["<|im_start|>", "<|im_end|>", "<think>", "</think>"]


def test_thinking_off_injects_an_empty_closed_span():
    tmpl = _HEAD + ("{% if add_generation_prompt %}<|im_start|>assistant\n"
                    "{% if enable_thinking is defined and enable_thinking is false %}<think>\n\n</think>\n\n{% endif %}"
                    "{% endif %}")
    p = derive_from_thinking_switch(_tok(tmpl, _SPECIALS))
    assert p is not None and (p.open, p.close, p.starts_open) == ("<think>", "</think>", False)


def test_thinking_off_swaps_the_opener_for_the_closer():
    tmpl = _HEAD + ("{% if add_generation_prompt %}<|im_start|>assistant\n"
                    "{% if enable_thinking is defined and enable_thinking is false %}</think>{% else %}<think>{% endif %}"
                    "{% endif %}")
    p = derive_from_thinking_switch(_tok(tmpl, _SPECIALS))
    assert (p.open, p.close, p.starts_open) == ("<think>", "</think>", True)


def test_both_renders_open_the_span():
    tmpl = _HEAD + ("{% if add_generation_prompt %}<|im_start|>assistant\n<think>\n"
                    "{% if enable_thinking is defined and enable_thinking is false %}\n</think>\n\n{% endif %}"
                    "{% endif %}")
    p = derive_from_tokenizer(_tok(tmpl, _SPECIALS))
    assert (p.open, p.close, p.starts_open) == ("<think>", "</think>", True)
    # the resolver prefers the tokenizer's evidence to a scan of the template text
    assert resolve_reasoning_parser("auto", "no delimiters in this text", _tok(tmpl, _SPECIALS)).close == "</think>"


def test_reasoning_as_a_separate_turn_gives_a_wildcard_closer_and_an_answer_header():
    specials = ["<|start|>", "<|eom|>", "<|message|>"]
    tmpl = ("{% for m in messages %}<|start|>{{ m.role }}"
            "{% if m.reasoning_content %} to=self<|message|>{{ m.reasoning_content }}<|eom|><|start|>assistant{% endif %}"
            " to=user<|message|>{{ m.content }}<|eom|>{% endfor %}"
            "{% if add_generation_prompt %}<|start|>assistant{% endif %}")
    tok = _tok(tmpl, specials)
    assert derive_from_thinking_switch(tok) is None          # no enable_thinking branch to compare
    p = derive_from_history(tok)
    assert p.open == "to=self<|message|>" and p.close == "<|eom|><|start|>assistant to=user<|message|>"
    assert (p.close_prefix, p.close_suffix) == ("<|eom|>", "<|message|>")
    assert p.answer_delim == " to=user<|message|>" and not p.starts_open


def test_a_template_without_reasoning_derives_nothing():
    tmpl = "{% for m in messages %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n{% endfor %}" \
           "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"
    assert derive_from_tokenizer(_tok(tmpl, _SPECIALS)) is None
