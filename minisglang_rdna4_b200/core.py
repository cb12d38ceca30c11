"""Request, batch and per-process context objects shared by the scheduler and the engine.

Semantics follow python/minisgl/core.py (SamplingParams :18-170, Req :173-268, Batch
:271-319, Context :322-377) with one structural change: the page table of this engine holds
real page ids (``[slot_row, position // page_size]``), not one entry per token, because the
sm_100a attention kernels fetch whole pages.
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Any, List, Literal, Optional

import torch

if TYPE_CHECKING:
    from .kvcache.base import BaseCacheHandle, BaseKVCachePool
    from .attention.base import AttnMetadata, BaseAttnBackend


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    min_p: float = 0.0
    ignore_eos: bool = False
    max_tokens: int = 1024
    logprobs: int = 0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    stop: List[str] = field(default_factory=list)
    stop_keep: List[str] = field(default_factory=list)
    grammar: Optional[str] = None
    grammar_required: bool = False
    # reasoning-span gate (a grammar engages only after the close delimiter was emitted)
    think_close_delim: Optional[str] = None
    think_answer_delim: Optional[str] = None
    think_close_prefix: Optional[str] = None
    think_close_suffix: Optional[str] = None
    think_tool_release: List[str] = field(default_factory=list)
    think_budget: int = 0
    think_span_open: bool = False
    # tool-call end-of-turn guard
    tool_call_openers: List[str] = field(default_factory=list)
    tool_call_closers: List[str] = field(default_factory=list)
    tool_match_gated: bool = False
    # keep the generated tokens in the prefix cache after the request ends
    cache_output: bool = True
    seed: Optional[int] = None

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    @property
    def has_penalty(self) -> bool:
        return self.presence_penalty != 0.0 or self.frequency_penalty != 0.0

    @property
    def constrained(self) -> bool:
        return self.grammar is not None


@dataclass(eq=False)
class Req:
    """One running sequence.

    ``cached_len`` tokens have their KV in the pool, ``device_len`` tokens exist (prompt plus
    committed output), and the next forward computes ``[cached_len, device_len)``. The
    invariant ``cached_len < device_len <= max_device_len`` always holds
    (python/minisgl/core.py:193-238).
    """

    input_ids: torch.Tensor  # 1-D int32 CPU tensor, a view of the preallocated host buffer
    table_idx: int
    cached_len: int
    output_len: int
    uid: int
    sampling_params: SamplingParams
    cache_handle: "BaseCacheHandle"

    def __post_init__(self) -> None:
        assert self.input_ids.device.type == "cpu"
        n = int(self.input_ids.numel())
        self.prompt_len = n
        self.device_len = n
        self.max_device_len = n + self.output_len
        assert 0 <= self.cached_len < self.device_len <= self.max_device_len, self
        buf = torch.empty(self.max_device_len, dtype=self.input_ids.dtype)
        buf[:n] = self.input_ids
        self._buf, self._len = buf, n
        self.input_ids = buf[:n]
        self.resources_freed = False
        self.finished = False
        self.finish_reason: Optional[str] = None

    # ---- lengths ----
    @property
    def remain_len(self) -> int:
        return self.max_device_len - self.device_len

    @property
    def extend_len(self) -> int:
        return self.device_len - self.cached_len

    @property
    def can_decode(self) -> bool:
        return self.remain_len > 0

    @property
    def generated_ids(self) -> torch.Tensor:
        return self._buf[self.prompt_len : self._len]

    @property
    def num_generated(self) -> int:
        return self._len - self.prompt_len

    # ---- state transitions ----
    def complete_one(self) -> None:
        """One forward finished: everything fed is cached and one new token now exists."""
        self.cached_len = self.device_len
        self.device_len += 1

    def complete_many(self, accepted: int) -> None:
        """A verify step committed ``accepted`` tokens (>= 1) at once."""
        assert accepted >= 1
        self.cached_len = self.device_len + accepted - 1
        self.device_len += accepted

    def append_host(self, tokens: torch.Tensor) -> None:
        n, end = self._len, self._len + int(tokens.numel())
        if end > self._buf.numel():
            grown = torch.empty(max(end, 2 * self._buf.numel()), dtype=self._buf.dtype)
            grown[:n] = self._buf[:n]
            self._buf = grown
        self._buf[n:end] = tokens
        self._len = end
        self.input_ids = self._buf[:end]

    def __repr__(self) -> str:
        return (
            f"Req(uid={self.uid}, slot={self.table_idx}, cached={self.cached_len}, "
            f"device={self.device_len}, max={self.max_device_len})"
        )


class ChunkedReq(Req):
    """A request whose prompt is only partly prefilled: never sampled, never decoded."""

    def append_host(self, tokens: torch.Tensor) -> None:  # pragma: no cover - guard
        raise RuntimeError("a partially prefilled request produces no token")

    @property
    def can_decode(self) -> bool:
        return False


@dataclass
class Batch:
    reqs: List[Req]
    phase: Literal["prefill", "decode"]
    # filled by the scheduler (device tensors)
    input_ids: torch.Tensor = field(init=False)
    positions: torch.Tensor = field(init=False)
    out_loc: torch.Tensor = field(init=False)
    padded_reqs: List[Req] = field(init=False)
    # filled by the attention backend
    attn_metadata: "AttnMetadata" = field(init=False)
    # a speculative verify batch is phase "decode" with extend_len = K+1 per request and
    # logits for every row; a custom additive mask selects tree verification
    spec_verify: bool = False
    verify_width: int = 0
    tree_mask: Optional[torch.Tensor] = None
    # the mask sliding-window layers take instead of ``tree_mask`` (a mask replaces their window rule too)
    tree_mask_swa: Optional[torch.Tensor] = None
    # > 0: ``tree_mask`` is ``[rows, mask_window]`` and covers the last mask_window K/V positions of each request
    mask_window: int = 0
    # capture the hidden states of these layer indices (EAGLE3 auxiliary features)
    capture_layers: Optional[List[int]] = None
    # sliding-window layers with a pool of their own: K/V slot of every row and block table in that pool
    # rows of this step whose embedding is given (image placeholder tokens) and the vectors that replace it
    mm_rows: Optional[torch.Tensor] = None
    mm_values: Optional[torch.Tensor] = None
    # a denoising step of a block-diffusion model with self-conditioning: the probability-weighted mean
    # embedding each canvas row predicted one step earlier, ``[rows, hidden]`` (zeros on a block's first step)
    canvas_signal: Optional[torch.Tensor] = None
    swa_out_loc: Optional[torch.Tensor] = None
    swa_block_table: Optional[torch.Tensor] = None

    def __post_init__(self) -> None:
        self.padded_reqs = self.reqs

    @property
    def is_prefill(self) -> bool:
        return self.phase == "prefill"

    @property
    def is_decode(self) -> bool:
        return self.phase == "decode"

    @property
    def size(self) -> int:
        return len(self.reqs)

    @property
    def padded_size(self) -> int:
        return len(self.padded_reqs)


@dataclass
class Context:
    """Per-process singleton that layers reach during a forward."""

    page_size: int
    page_table: torch.Tensor = field(init=False)      # [slots, max_pages] int32, page ids
    attn_backend: "BaseAttnBackend" = field(init=False)
    kv_cache: "BaseKVCachePool" = field(init=False)
    moe_backend: Any = None
    ep: Any = None
    comm: Any = None
    aux_hidden: Optional[List[torch.Tensor]] = None
    # recurrent state of gated-delta-net layers (kvcache.gdn_state.GDNStateCache), hybrid models only
    # K/V pool of the sliding-window layers when they have one of their own (kvcache.swa_pages)
    swa_kv_cache: Any = None
    gdn_state: Any = None
    # speculative verify of a hybrid model: every recurrent layer appends (layer, its projected step
    # input) here, so that the state can be rebuilt for the accepted rows only (list, or None = off)
    recurrent_journal: Any = None
    _batch: Optional[Batch] = None

    @property
    def batch(self) -> Batch:
        assert self._batch is not None, "no forward is active"
        return self._batch

    @contextmanager
    def forward_batch(self, batch: Batch):
        assert self._batch is None, "forward_batch does not nest"
        self._batch = batch
        try:
            yield
        finally:
            self._batch = None


_CTX: Optional[Context] = None


def set_global_ctx(ctx: Optional[Context]) -> None:
    global _CTX
    _CTX = ctx


def get_global_ctx() -> Context:
    assert _CTX is not None, "global context is not set"
    return _CTX


def try_global_ctx() -> Optional[Context]:
    return _CTX
