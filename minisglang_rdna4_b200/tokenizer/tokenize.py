"""Prompt rendering and tokenisation (python/minisgl/tokenizer/tokenize.py:15-120): plain
strings are encoded as they are; chat message lists go through the tokenizer's chat template
with the request's template kwargs and tool definitions, falling back to progressively
simpler calls for templates that reject an argument."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch


class TokenizeManager:
    def __init__(self, tokenizer, chat_template: Optional[str] = None,
                 default_kwargs: Optional[Dict[str, Any]] = None) -> None:
        self.tokenizer = tokenizer
        self.chat_template = chat_template
        self.default_kwargs = dict(default_kwargs or {})

    def render(self, messages: List[Dict[str, Any]], kwargs: Optional[Dict[str, Any]] = None,
               tools: Optional[List[Dict[str, Any]]] = None, add_generation_prompt: bool = True) -> str:
        kw = dict(self.default_kwargs)
        kw.update(kwargs or {})
        attempts = []
        base = dict(tokenize=False, add_generation_prompt=add_generation_prompt)
        if self.chat_template:
            base["chat_template"] = self.chat_template
        if tools:
            attempts.append(dict(base, tools=tools, **kw))
        attempts.append(dict(base, **kw))
        attempts.append(dict(base))
        last: Optional[Exception] = None
        for args in attempts:
            try:
                return self.tokenizer.apply_chat_template(messages, **args)
            except Exception as exc:  # template rejected an argument: retry with fewer
                last = exc
        raise ValueError(f"chat template failed: {last}")

    def tokenize(self, text_or_messages: Any, kwargs=None, tools=None, add_generation_prompt=True) -> torch.Tensor:
        if isinstance(text_or_messages, str):
            ids = self.tokenizer.encode(text_or_messages)
        elif isinstance(text_or_messages, (list, tuple)) and text_or_messages and isinstance(text_or_messages[0], int):
            ids = list(text_or_messages)
        else:
            text = self.render(list(text_or_messages), kwargs, tools, add_generation_prompt)
            ids = self.tokenizer.encode(text, add_special_tokens=False) if _accepts_special(self.tokenizer) \
                else self.tokenizer.encode(text)
        return torch.tensor(ids, dtype=torch.int32)


def _accepts_special(tok) -> bool:
    try:
        import inspect

        return "add_special_tokens" in inspect.signature(tok.encode).parameters
    except (TypeError, ValueError):
        return True
