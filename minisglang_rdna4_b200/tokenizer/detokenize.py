"""Incremental detokenisation with stop strings
(python/minisgl/tokenizer/detokenize.py:78-214).

Text is emitted only when it is stable: a trailing replacement character (an incomplete
UTF-8 sequence) or a tail that could still grow into a stop string is held back. ``stop``
strings end the request and are trimmed from the output; ``stop_keep`` strings end it and
stay in the output.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class _State:
    ids: List[int] = field(default_factory=list)
    prefix_offset: int = 0     # ids[prefix_offset:read_offset] is the context already emitted
    read_offset: int = 0
    text: str = ""             # everything decoded so far
    sent: int = 0              # characters of `text` already sent
    stop: List[str] = field(default_factory=list)
    stop_keep: List[str] = field(default_factory=list)
    done: bool = False


class DetokenizeManager:
    def __init__(self, tokenizer) -> None:
        self.tokenizer = tokenizer
        self.states: Dict[int, _State] = {}

    def register(self, uid: int, stop: List[str], stop_keep: List[str]) -> None:
        self.states[uid] = _State(stop=list(stop or []), stop_keep=list(stop_keep or []))

    def _decode_new(self, st: _State) -> str:
        tok = self.tokenizer
        prefix = tok.decode(st.ids[st.prefix_offset:st.read_offset], skip_special_tokens=True)
        full = tok.decode(st.ids[st.prefix_offset:], skip_special_tokens=True)
        if full.endswith("�"):
            return ""  # incomplete multi-byte character: wait for more tokens
        new = full[len(prefix):]
        st.prefix_offset = st.read_offset
        st.read_offset = len(st.ids)
        return new

    def step(self, uid: int, token: int, finished: bool) -> Tuple[str, bool, Optional[str]]:
        """Feed one token. Returns ``(text to send, stop string hit, which)``."""
        st = self.states.get(uid)
        if st is None:
            st = self.states[uid] = _State()
        if st.done:
            return "", False, None
        st.ids.append(int(token))
        st.text += self._decode_new(st)
        hit, which, cut = False, None, len(st.text)
        for s in st.stop:
            pos = st.text.find(s, max(0, st.sent - len(s)))
            if pos != -1 and pos < cut:
                hit, which, cut = True, s, pos
        for s in st.stop_keep:
            pos = st.text.find(s, max(0, st.sent - len(s)))
            if pos != -1 and pos + len(s) <= cut:
                hit, which, cut = True, s, pos + len(s)
        if hit:
            out = st.text[st.sent:cut]
            st.sent = cut
            st.done = True
            return out, True, which
        if finished:
            if st.read_offset < len(st.ids):  # flush whatever is still pending
                st.text += self.tokenizer.decode(st.ids[st.prefix_offset:], skip_special_tokens=True)[
                    len(self.tokenizer.decode(st.ids[st.prefix_offset:st.read_offset], skip_special_tokens=True)):]
            out = st.text[st.sent:]
            st.sent = len(st.text)
            st.done = True
            return out, False, None
        # hold back a tail that is a proper prefix of some stop string
        hold = 0
        for s in st.stop + st.stop_keep:
            for k in range(min(len(s) - 1, len(st.text) - st.sent), 0, -1):
                if st.text.endswith(s[:k]):
                    hold = max(hold, k)
                    break
        end = len(st.text) - hold
        out = st.text[st.sent:end] if end > st.sent else ""
        st.sent = max(st.sent, end)
        return out, False, None

    def finish(self, uid: int) -> None:
        self.states.pop(uid, None)
