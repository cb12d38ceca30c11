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
    # templates that route reasoning and answer as separate turns: the header the model writes when it
    # answers directly, and a closer whose middle names a recipient (prefix .. anything .. suffix)
    answer_delim: Optional[str] = None
    close_prefix: Optional[str] = None
    close_suffix: Optional[str] = None
    how: str = ""                 # where the delimiters came from (for the boot log)

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


# ---------------------------------------------------------------------------- derivation from a tokenizer
_PROBE = [{"role": "user", "content": "hi"}]
_RSN_MARK, _ANS_MARK = "ZQREASONINGZQ", "ZQANSWERZQ"
_HISTORY_PROBE = [{"role": "user", "content": "hi"},
                  {"role": "assistant", "reasoning_content": _RSN_MARK, "content": _ANS_MARK}]
_DELIM_RE = re.compile(r"<\|[^|<>\n]{1,48}\|>|<[^<>\s|]{1,48}\|>|<\|[^<>\s|]{1,48}>|</?[A-Za-z_][\w:\-]{0,47}>|◁[^▷\n]{1,32}▷")


def _render(tokenizer, messages, gen: bool, **kw) -> Optional[str]:
    try:
        return tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=gen, **kw)
    except Exception:
        return None


def _delim_chunks(tokenizer, text: str) -> List[Tuple[str, bool]]:
    """``text`` cut into ``(piece, is_delimiter)``: a delimiter is one of the tokenizer's added
    tokens with a non-blank surface, or (no tokenizer vocabulary) something tag-shaped. Cutting at
    delimiter level, not character level, keeps ``<think>`` and ``</think>`` from sharing a ``<``."""
    added = set()
    try:
        added = {t for t in tokenizer.get_added_vocab() if len(t.strip()) >= 2}
    except Exception:
        pass
    if added:
        pat = re.compile("|".join(re.escape(t) for t in sorted(added, key=len, reverse=True)))
    else:
        pat = _DELIM_RE
    out, pos = [], 0
    for m in pat.finditer(text):
        if m.start() > pos:
            out.append((text[pos:m.start()], False))
        out.append((m.group(0), True))
        pos = m.end()
    if pos < len(text):
        out.append((text[pos:], False))
    return out


def _tail(tokenizer, messages, **kw) -> Optional[str]:
    """What ``add_generation_prompt`` appends to the rendered conversation."""
    with_p, without = _render(tokenizer, messages, True, **kw), _render(tokenizer, messages, False, **kw)
    if with_p is None or without is None:
        return None
    return with_p[len(without):] if with_p.startswith(without) else with_p


def derive_from_thinking_switch(tokenizer) -> Optional[ReasoningParser]:
    """Render the generation-prompt tail with ``enable_thinking`` on and off and compare them at
    delimiter level. "Thinking off" is spelled by ending the span inside the prompt, so the last
    delimiter that only the off-tail has is the closer. The opener is read, most direct evidence
    first, from (a) an empty pre-closed span in the off-tail, (b) what only the on-tail has (the
    template swaps opener for closer), (c) the last delimiter the two tails share
    (python/minisgl/server/reasoning.py:654-735)."""
    on, off = _tail(tokenizer, _PROBE, enable_thinking=True), _tail(tokenizer, _PROBE, enable_thinking=False)
    if on is None or off is None or on == off:
        return None
    on_c, off_c = _delim_chunks(tokenizer, on), _delim_chunks(tokenizer, off)
    i = 0
    while i < min(len(on_c), len(off_c)) and on_c[i] == off_c[i]:
        i += 1
    on_mid, off_mid = on_c[i:], off_c[i:]
    on_delims = {t for t, d in on_mid if d}
    closers = [k for k, (t, d) in enumerate(off_mid) if d and t not in on_delims]
    if not closers:
        return None
    ci = closers[-1]
    close = off_mid[ci][0]
    pre = [t for t, d in off_mid[:ci] if d]
    if pre:
        # the opener may carry a channel name the closer does not: keep the text up to the closer
        opener = "".join(t for t, _ in off_mid[:ci]).strip()
        return ReasoningParser(opener, close, False, how="chat template: thinking-off injects an empty closed span")
    on_text = "".join(t for t, _ in on_mid).strip()
    if on_text and on_delims:
        return ReasoningParser(on_text, close, True, how="chat template: thinking-off swaps the opener for the closer")
    for t, d in reversed(on_c[:i]):
        if d and t != close:
            return ReasoningParser(t, close, True, how="chat template: opener common to both renders")
    return None


def derive_from_history(tokenizer) -> Optional[ReasoningParser]:
    """Render an assistant turn that carries reasoning and read the delimiters around the two
    markers: whatever stands between reasoning and answer is the closer (several delimiters when the
    template routes them as separate turns, in which case the first and last form a wildcard and the
    part after the assistant header is the direct-answer header); the opener is what the template
    writes between the assistant header and the reasoning
    (python/minisgl/server/reasoning.py:738-905)."""
    text = _render(tokenizer, _HISTORY_PROBE, False)
    if text is None or _RSN_MARK not in text or _ANS_MARK not in text:
        return None
    r0, a0 = text.index(_RSN_MARK), text.index(_ANS_MARK)
    if a0 < r0:
        return None
    between = text[r0 + len(_RSN_MARK):a0]
    mids = [t for t, d in _delim_chunks(tokenizer, between) if d]
    if not mids:
        return None
    head = _tail(tokenizer, _PROBE) or ""
    before = text[:r0]
    hdr = head.strip()
    opener = before[before.rindex(hdr) + len(hdr):] if hdr and hdr in before else ""
    open_delims = [t for t, d in _delim_chunks(tokenizer, opener) if d]
    if not open_delims:
        cands = [t for t, d in _delim_chunks(tokenizer, before) if d]
        if not cands:
            return None
        opener = cands[-1]
    close = between.strip()
    starts_open = bool(opener.strip()) and head.rstrip().endswith(opener.strip())
    extra = {}
    if len(mids) >= 3:
        extra = dict(close_prefix=mids[0], close_suffix=mids[-1])
        if hdr and hdr in close:
            answer = close[close.index(hdr) + len(hdr):]
            if answer.strip():
                extra["answer_delim"] = answer
    return ReasoningParser(opener.strip(), close, starts_open, how="chat template: assistant turn with reasoning", **extra)


def derive_from_tokenizer(tokenizer) -> Optional[ReasoningParser]:
    if tokenizer is None or not getattr(tokenizer, "chat_template", None):
        return None
    return derive_from_thinking_switch(tokenizer) or derive_from_history(tokenizer)


def resolve_reasoning_parser(name: str, chat_template: Optional[str], tokenizer=None) -> Optional[ReasoningParser]:
    """``auto`` derives the delimiters (from the tokenizer's rendered template when one is given,
    else from the template text), ``none`` disables the split, a known name selects a fixed pair."""
    if name in (None, "none", "off"):
        return None
    if name == "auto":
        return derive_from_tokenizer(tokenizer) or derive_delimiters(chat_template)
    if name in NAMED_PARSERS:
        o, c = NAMED_PARSERS[name]
        derived = derive_from_tokenizer(tokenizer) or derive_delimiters(chat_template)
        return ReasoningParser(o, c, derived.starts_open if derived and derived.open == o else False)
    raise ValueError(f"unknown reasoning parser {name!r}; choices: auto, none, {', '.join(sorted(NAMED_PARSERS))}")
