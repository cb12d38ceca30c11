"""Reasoning-span handling: find a model's think delimiters and split generated text into
``reasoning_content`` and ``content``, incrementally for streaming
(python/minisgl/server/reasoning.py:162 ReasoningParser, :360 ReasoningStreamState, :654
derive_delimiters, :912 resolve_reasoning_parser)."""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import List, Optional, Tuple

# (open, close) pairs seen in public chat templates, most specific first
KNOWN_DELIMITERS: Tuple[Tuple[str, str], ...] = (
    ("<think>", "</think>"),
    ("<|begin_of_thought|>", "<|end_of_thought|>"),
    ("<reasoning>", "</reasoning>"),
    ("<|channel|>analysis<|message|>", "<|end|>"),
    ("◁think▷", "◁/think▷"),
)
NAMED_PARSERS = {
    "qwen3": ("<think>", "</think>"), "deepseek-r1": ("<think>", "</think>"), "glm": ("<think>", "</think>"),
    "think": ("<think>", "</think>"), "gpt-oss": ("<|channel|>analysis<|message|>", "<|end|>"),
}


@dataclass(frozen=True)
class ReasoningParser:
    open: str
    close: str
    # the generation prompt of the template ends inside the span (the model starts by thinking)
    starts_open: bool = False

    def split(self, text: str, thinking_open: Optional[bool] = None) -> Tuple[Optional[str], str]:
        """Whole-text split: ``(reasoning or None, content)``."""
        is_open = self.starts_open if thinking_open is None else thinking_open
        st = ReasoningStreamState(self, is_open)
        r, c = st.feed(text)
        r2, c2 = st.flush()
        reasoning, content = r + r2, c + c2
        return (reasoning if reasoning else None), content


class ReasoningStreamState:
    """Incremental splitter. ``feed`` returns ``(reasoning delta, content delta)``; text that
    may be the beginning of a delimiter is held back until it is decided."""

    def __init__(self, parser: ReasoningParser, thinking_open: bool = False) -> None:
        self.p = parser
        self.in_think = thinking_open
        self.closed = False          # a span was closed: later open tags are plain content
        self.buf = ""

    def _hold(self, text: str, delim: str) -> int:
        for k in range(min(len(delim) - 1, len(text)), 0, -1):
            if text.endswith(delim[:k]):
                return k
        return 0

    def feed(self, delta: str) -> Tuple[str, str]:
        self.buf += delta
        reasoning, content = [], []
        while True:
            if self.in_think:
                pos = self.buf.find(self.p.close)
                if pos != -1:
                    reasoning.append(self.buf[:pos])
                    self.buf = self.buf[pos + len(self.p.close):].lstrip("\n") if True else ""
                    self.in_think, self.closed = False, True
                    continue
                hold = self._hold(self.buf, self.p.close)
                cut = len(self.buf) - hold
                reasoning.append(self.buf[:cut])
                self.buf = self.buf[cut:]
                break
            if not self.closed:
                pos = self.buf.find(self.p.open)
                if pos != -1:
                    content.append(self.buf[:pos])
                    self.buf = self.buf[pos + len(self.p.open):]
                    self.in_think = True
                    continue
                hold = self._hold(self.buf, self.p.open)
                cut = len(self.buf) - hold
                content.append(self.buf[:cut])
                self.buf = self.buf[cut:]
                break
            content.append(self.buf)
            self.buf = ""
            break
        return "".join(reasoning), "".join(content)

    def flush(self) -> Tuple[str, str]:
        out = self.buf
        self.buf = ""
        return (out, "") if self.in_think else ("", out)


def derive_delimiters(chat_template: Optional[str]) -> Optional[ReasoningParser]:
    """Look for a known delimiter pair in the template text and decide whether the generation
    prompt leaves the span open (the template emits the open tag after the assistant header
    when ``add_generation_prompt`` is set)."""
    if not chat_template:
        return None
    for open_, close in KNOWN_DELIMITERS:
        if close in chat_template or open_ in chat_template:
            starts_open = False
            m = re.search(r"add_generation_prompt(.{0,400})", chat_template, re.S)
            if m and open_ in m.group(1) and close not in m.group(1).split(open_, 1)[1][:40]:
                starts_open = True
            return ReasoningParser(open_, close, starts_open)
    return None


def resolve_reasoning_parser(name: str, chat_template: Optional[str]) -> Optional[ReasoningParser]:
    """``auto`` derives the delimiters from the template, ``none`` disables the split, a known
    name selects a fixed pair."""
    if name in (None, "none", "off"):
        return None
    if name == "auto":
        return derive_delimiters(chat_template)
    if name in NAMED_PARSERS:
        o, c = NAMED_PARSERS[name]
        derived = derive_delimiters(chat_template)
        return ReasoningParser(o, c, derived.starts_open if derived and derived.open == o else False)
    raise ValueError(f"unknown reasoning parser {name!r}; choices: auto, none, {', '.join(sorted(NAMED_PARSERS))}")
