"""Chunked-prefill packing under a per-step token budget
(python/minisgl/scheduler/prefill.py:43-276).

Rules kept from the reference: FIFO admission that stops at the first request that does not
fit; admission needs ``extend + output + reserved <= free + evictable`` both before and
after locking the matched prefix; a chunk that does not finish its prompt leaves 256 tokens
of the budget to requests queued behind it when the budget exceeds 512; a partially
prefilled request stays at the head of the queue and is never sampled.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from ..core import Batch, ChunkedReq, Req, SamplingParams
from .cache import CacheManager
from .decode import DecodeManager
from .table import TableManager

SHORT_REQ_RESERVE = 256
MIN_CHUNK = 256


@dataclass
class PendingReq:
    uid: int
    input_ids: torch.Tensor
    sampling_params: SamplingParams
    chunked: Optional[ChunkedReq] = None
    spans: Optional[object] = None          # [n, 2] positions of image placeholder runs

    @property
    def input_len(self) -> int:
        return int(self.input_ids.numel())

    @property
    def output_len(self) -> int:
        return self.sampling_params.max_tokens


class PrefillAdder:
    def __init__(self, token_budget: int, reserved_tokens: int, cache: CacheManager,
                 table: TableManager, others_waiting: int = 0) -> None:
        self.token_budget = token_budget
        self.reserved = reserved_tokens
        self.cache = cache
        self.table = table
        self.others_waiting = others_waiting
        self.new_slots: List[Tuple[int, torch.Tensor, int]] = []  # (slot, prompt ids, cached_len)
        self.restores: List[Tuple[int, int]] = []                 # (slot, recurrent-state snapshot id)

    def _chunk(self, remain: int) -> int:
        chunk = min(self.token_budget, remain)
        if chunk < remain and self.others_waiting > 0 and self.token_budget > 2 * SHORT_REQ_RESERVE:
            chunk = max(MIN_CHUNK, chunk - SHORT_REQ_RESERVE)
        return chunk

    def try_add(self, pending: PendingReq) -> Optional[Req]:
        if self.token_budget <= 0:
            return None
        ps = self.cache.page_size
        if pending.chunked is not None:
            prev = pending.chunked
            slot, handle, cached = prev.table_idx, prev.cache_handle, prev.cached_len
            # an admitted request still owes pages for the rest of its prompt and for its output:
            # requests admitted behind it in this step must not count that room as theirs
            # (python/minisgl/scheduler/prefill.py:160 reserves remain + output for every request)
            self.reserved += pending.input_len - cached + pending.output_len
        else:
            if self.table.available_size == 0:
                return None
            handle, pages = self.cache.match_req(pending.input_ids)
            cached = handle.cached_len
            need = pending.input_len - cached + pending.output_len
            if need + self.reserved > self.cache.available_tokens:
                return None
            self.cache.lock(handle)
            if need + self.reserved > self.cache.available_tokens:
                self.cache.unlock(handle)
                return None
            slot = self.table.allocate()
            self.cache.set_prefix_pages(slot, pages)
            self.cache.prefix_hit_tokens += cached
            self.cache.prefix_query_tokens += pending.input_len
            self.new_slots.append((slot, pending.input_ids, cached))
            if getattr(handle, "snap", None) is not None:
                self.restores.append((slot, handle.snap))     # recurrent state to copy into the slot
            self.reserved += need
        remain = pending.input_len - cached
        chunk = self._chunk(remain)
        if chunk < remain and (cached + chunk) % ps and chunk > (cached + chunk) % ps:
            # a chunk that is not the last ends on a page boundary: recurrent-state snapshots and the
            # prefix cache work in whole pages
            chunk -= (cached + chunk) % ps
        spans = getattr(pending, "spans", None)
        if spans is not None and chunk < remain:
            # the tokens of one image are computed in one step (they attend to each other): a chunk that
            # would end inside an image stops before it, or takes all of it when the image comes first
            end = cached + chunk
            for a, b in spans.tolist():
                if a < end < b:
                    chunk = (a - cached) if a > cached else min(remain, b - cached)
                    break
        self.token_budget -= chunk
        final = chunk == remain
        cls = Req if final else ChunkedReq
        req = cls(
            input_ids=pending.input_ids[: cached + chunk], table_idx=slot, cached_len=cached,
            output_len=pending.output_len if final else pending.input_len - (cached + chunk) + pending.output_len,
            uid=pending.uid, sampling_params=pending.sampling_params, cache_handle=handle,
        )
        if final:
            # the request object that lives on: full prompt, output budget
            req.max_device_len = pending.input_len + pending.output_len
        pending.chunked = None if final else req  # type: ignore[assignment]
        return req


class PrefillManager:
    def __init__(self, cache: CacheManager, table: TableManager, decode: DecodeManager) -> None:
        self.cache, self.table, self.decode = cache, table, decode
        self.pending: List[PendingReq] = []

    def add_one_req(self, uid: int, input_ids: torch.Tensor, params: SamplingParams) -> None:
        self.pending.append(PendingReq(uid, input_ids, params))

    def abort(self, uid: int) -> Optional[PendingReq]:
        for i, p in enumerate(self.pending):
            if p.uid == uid:
                return self.pending.pop(i)
        return None

    @property
    def runnable(self) -> bool:
        return bool(self.pending)

    def schedule_next_batch(self, token_budget: int):
        """Returns ``(batch, adder)`` or ``(None, None)``."""
        if not self.pending:
            return None, None
        adder = PrefillAdder(token_budget, self.decode.inflight_tokens, self.cache, self.table,
                             others_waiting=len(self.pending) - 1)
        reqs: List[Req] = []
        done = 0
        for pending in self.pending:
            req = adder.try_add(pending)
            if req is None:
                break
            reqs.append(req)
            if pending.chunked is not None:
                break  # the partially prefilled request keeps the head of the queue
            done += 1
        if not reqs:
            return None, None
        self.pending = self.pending[done:]
        # longest extend first: the attention grid walks requests in batch order and the long ones
        # have the most work per query tile (admission order only decided who got into the step)
        reqs.sort(key=lambda r: (-(r.device_len - r.cached_len), r.uid))
        return Batch(reqs=reqs, phase="prefill"), adder
