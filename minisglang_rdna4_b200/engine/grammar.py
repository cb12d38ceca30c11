"""Structured output: xgrammar compilation and per-step token bitmasks
(python/minisgl/engine/grammar.py:27-100).

A request's ``grammar`` field is ``"json"`` (any JSON value), a JSON-schema string, or an EBNF
grammar prefixed with ``ebnf:``. The scheduler keeps one matcher per constrained request,
fills a ``[n, ceil(V/32)]`` int32 bitmask for the rows that are constrained this step, and
advances each matcher with the token that was committed. When a request has a reasoning span
the grammar only engages after the close delimiter (``ThinkGate``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


class GrammarBackend:
    def __init__(self, tokenizer=None, vocab_size: Optional[int] = None, stop_token_ids: Optional[List[int]] = None,
                 encoded_vocab: Optional[List[bytes]] = None) -> None:
        import xgrammar as xgr

        self.xgr = xgr
        if encoded_vocab is not None:
            info = xgr.TokenizerInfo(encoded_vocab, vocab_size=vocab_size, stop_token_ids=stop_token_ids)
        else:
            from ..tokenizer.simple import ByteTokenizer

            if isinstance(tokenizer, ByteTokenizer) or tokenizer is None:
                tok = tokenizer or ByteTokenizer()
                vocab = [bytes([i]) for i in range(256)] + [f"<|{i}|>".encode() for i in range(256, tok.vocab_size)]
                vs = vocab_size or tok.vocab_size
                vocab = vocab + [f"<|pad{i}|>".encode() for i in range(len(vocab), vs)]
                info = xgr.TokenizerInfo(vocab[:vs], vocab_size=vs, stop_token_ids=stop_token_ids or [tok.eos_token_id])
            else:
                info = xgr.TokenizerInfo.from_huggingface(tokenizer, vocab_size=vocab_size,
                                                          stop_token_ids=stop_token_ids)
        self.info = info
        self.vocab_size = info.vocab_size
        self.compiler = xgr.GrammarCompiler(info, max_threads=4)
        self._cache: Dict[str, object] = {}

    def compile(self, spec: str):
        hit = self._cache.get(spec)
        if hit is not None:
            return hit
        if spec == "json":
            compiled = self.compiler.compile_builtin_json_grammar()
        elif spec.startswith("ebnf:"):
            compiled = self.compiler.compile_grammar(spec[5:])
        elif spec.startswith("structural_tag:"):
            compiled = self.compiler.compile_structural_tag(spec[len("structural_tag:"):])
        else:
            compiled = self.compiler.compile_json_schema(spec)
        self._cache[spec] = compiled
        return compiled

    def new_matcher(self, spec: str):
        return self.xgr.GrammarMatcher(self.compile(spec))

    def allocate_bitmask(self, rows: int) -> torch.Tensor:
        return self.xgr.allocate_token_bitmask(rows, self.vocab_size)

    def fill(self, matcher, bitmask: torch.Tensor, row: int) -> None:
        matcher.fill_next_token_bitmask(bitmask, row)


class GrammarState:
    """Per-scheduler bookkeeping of the matchers of constrained requests."""

    def __init__(self, backend: GrammarBackend) -> None:
        self.backend = backend
        self.matchers: Dict[int, object] = {}

    def ensure(self, uid: int, spec: str):
        m = self.matchers.get(uid)
        if m is None:
            m = self.matchers[uid] = self.backend.new_matcher(spec)
        return m

    def build_bitmask(self, uids: Sequence[int], specs: Sequence[Optional[str]], active: Sequence[bool]):
        """Returns ``(bitmask [n_constrained, W] int32 CPU, rows)`` or ``(None, None)``."""
        rows = [i for i, (s, a) in enumerate(zip(specs, active)) if s is not None and a]
        if not rows:
            return None, None
        bm = self.backend.allocate_bitmask(len(rows))
        for j, i in enumerate(rows):
            m = self.ensure(uids[i], specs[i])
            if m.is_terminated():
                # grammar complete: only the stop tokens stay allowed (fill handles it)
                pass
            self.backend.fill(m, bm, j)
        return bm, torch.tensor(rows, dtype=torch.int64)

    def accept(self, uid: int, token: int) -> bool:
        m = self.matchers.get(uid)
        if m is None or m.is_terminated():
            return True
        return bool(m.accept_token(int(token)))

    def finish(self, uid: int) -> None:
        self.matchers.pop(uid, None)
