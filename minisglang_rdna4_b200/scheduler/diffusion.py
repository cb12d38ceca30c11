"""Block-diffusion execution: the scheduler loop and the per-request canvas bookkeeping
(python/minisgl/scheduler/diffusion.py:56-614).

A block-diffusion request does not emit one token per forward. It cycles

    encode   one causal forward over tokens that have no K/V yet (the prompt, later the block that
             was just committed); nothing is sampled from it
    denoise  up to ``max_steps`` forwards over a canvas of ``block`` positions behind the committed
             text; the canvas rows see the committed K/V and each other in both directions;
             nothing is emitted, the canvas state advances (``diffusion.sampler.Canvas``)
    commit   the block's candidate tokens are emitted at once (cut at an end-of-sequence token or
             the token budget) and become text that needs encoding

The canvas lives in the K/V slots the committed block will occupy: every denoising forward
rewrites them with bidirectional K/V and the encode pass after the commit rewrites them once more
with the causal K/V the next block reads. No scratch pool, and the request's page-table row stays
a plain prefix that the prefix cache can take over when the request ends. Request lengths
(``cached_len`` / ``device_len``) only move at commits, never between denoising steps.

Prompts are admitted and chunked by the ordinary prefill manager (prefix-cache hits included); its
final chunk is run without a sampled row. Denoising rows go through the engine's verification
path: a zero additive mask over the last ``block`` K/V positions replaces the causal rule for
those rows (``Batch.mask_window``), which is the attention form the tree-verification step uses.
Sliding-window layers take a second mask (the canvas whole, committed text inside the row's window); the
window rule for positions the masks do not cover is applied by the tensor-op attention path only, so such
models are refused on a GPU.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..core import Batch, Req
from ..diffusion import Canvas, DenoiseConfig
from ..engine import BatchSamplingArgs
from ..message import DetokenizeMsg
from ..utils import init_logger
from .prefill import ChunkedReq

logger = init_logger(__name__)


class CanvasManager:
    """Denoising state per request id. Allocated when a block opens, dropped when it is committed;
    freeing is idempotent (finish, abort and commit can all reach a request)."""

    def __init__(self, cfg: DenoiseConfig, device, seed: int) -> None:
        self.cfg, self.device, self.seed = cfg, torch.device(device), int(seed)
        self._state: Dict[int, Canvas] = {}
        self._gen: Dict[int, torch.Generator] = {}
        self.steps_per_block: List[int] = []

    def get(self, uid: int) -> Optional[Canvas]:
        return self._state.get(uid)

    def begin(self, uid: int, length: int, seed: Optional[int]) -> Canvas:
        gen = self._gen.get(uid)
        if gen is None:
            # one generator per request, kept across its blocks (a generator per block would replay the
            # first block's noise in the second); the same seed on every tensor-parallel rank
            gen = torch.Generator(device=self.device)
            gen.manual_seed(int(seed) if seed is not None else (self.seed * 1_000_003 + uid) & 0x7FFFFFFF)
            self._gen[uid] = gen
        st = Canvas(self.cfg, length, self.device, gen)
        self._state[uid] = st
        return st

    def end(self, uid: int) -> None:
        st = self._state.pop(uid, None)
        if st is not None:
            self.steps_per_block.append(st.steps_taken)

    def free(self, uid: int) -> None:
        self._state.pop(uid, None)
        self._gen.pop(uid, None)

    @property
    def num_active(self) -> int:
        return len(self._state)


def make_canvas_manager(sched) -> Optional[CanvasManager]:
    eng = sched.engine
    mc = eng.model_config
    if not mc.canvas_length:
        return None
    if mc.is_recurrent:
        raise ValueError("block-diffusion decoding needs a model without recurrent layers")
    if mc.swa_layers and (eng.device.type == "cuda" or eng.swa is not None):
        # canvas rows of a sliding-window layer see the whole canvas and the text inside their window: a
        # second mask plus the window rule for the positions the mask does not cover, which only the
        # tensor-op attention path applies
        raise ValueError("block-diffusion decoding with sliding-window layers runs on the CPU oracle path only "
                         "(and without the sliding-window pool)")
    if sched.config.spec_algorithm != "none":
        raise ValueError("block-diffusion decoding and speculative decoding exclude each other")
    cfg = DenoiseConfig.from_model(sched.config.model_path, mc, getattr(sched.config, "diffusion_overrides", None))
    logger.info_rank0("block diffusion: %s rule, %d-token blocks, up to %d steps per block", cfg.kind, cfg.block,
                      cfg.max_steps)
    return CanvasManager(cfg, eng.device, sched.config.seed)


def _no_sample(plan):
    plan.sample_rows = np.zeros(0, dtype=np.int32)
    plan.write_idx = np.zeros(0, dtype=np.int32)
    return plan


def _encode(sched, reqs: List[Req]) -> None:
    """Causal forward over ``[cached_len, device_len)`` of every request; K/V only."""
    if not reqs:
        return
    batch = Batch(reqs=reqs, phase="prefill")
    plan = _no_sample(sched._make_plan(batch))
    sched.engine.forward_batch(batch, plan, BatchSamplingArgs())
    sched.stats["steps"] += 1
    sched.stats["prefill_tokens"] += plan.num_tokens
    for r in reqs:
        r.cached_len = r.device_len                # everything fed has causal K/V now


def _denoise(sched, mgr: CanvasManager, reqs: List[Req]) -> None:
    """One denoising forward over the open canvases of ``reqs`` and the state update of each."""
    eng = sched.engine
    msl = sched.max_seq_len
    lens = [mgr.get(r.uid).length for r in reqs]
    width = max(lens)
    pool = eng.token_pool.view(-1)
    # the canvas tokens are the input of this forward: they go behind the committed text in the token pool
    idx = torch.cat([torch.arange(r.table_idx * msl + r.device_len, r.table_idx * msl + r.device_len + n)
                     for r, n in zip(reqs, lens)])
    tok = torch.cat([mgr.get(r.uid).tokens for r in reqs]).to(torch.int32)
    batch = Batch(reqs=reqs, phase="decode")
    batch.spec_verify = True                       # every row yields logits, nothing is written back
    # _make_plan feeds (device_len - cached_len) + extra rows per request: here cached_len == device_len
    # and the extra rows are the canvas. Requests with a shorter (last) block get a plan of their own width.
    if len(set(lens)) == 1:
        plan = sched._make_plan(batch, extra_rows=width)
    else:
        plan = _ragged_plan(sched, batch, lens)
    total = plan.num_tokens
    # zero bias over the last `width` K/V positions of every request: its canvas (all of it, in both
    # directions) and, for a shorter last block, the committed text just ahead of it
    window = int(eng.model_config.sliding_window or 0) if eng.model_config.swa_layers else 0
    span = width + window                          # K/V positions the masks cover
    mask = torch.zeros((total, span), dtype=torch.float32)
    mask_swa = None
    cu = plan.cu_q.tolist()
    if window:
        # sliding-window layers: the canvas in both directions, committed text only inside the row's window
        mask_swa = torch.zeros((total, span), dtype=torch.float32)
        for i, (r, n) in enumerate(zip(reqs, lens)):
            kv_len = r.device_len + n
            k_pos = torch.arange(kv_len - span, kv_len)[None, :]
            q_pos = torch.arange(r.device_len, kv_len)[:, None]
            hidden = (k_pos < r.device_len) & (k_pos <= q_pos - window)
            mask_swa[cu[i]:cu[i + 1]] = torch.where(hidden, float("-inf"), 0.0)
    soft = getattr(eng.model, "soft_embedding", None)
    stream_ctx = torch.cuda.stream(eng.stream) if eng.stream is not None else _null()
    with stream_ctx:
        pool[idx.to(eng.device, non_blocking=True)] = tok.to(eng.device, non_blocking=True)
        batch.tree_mask = mask.to(eng.device)
        batch.tree_mask_swa = mask_swa.to(eng.device) if mask_swa is not None else None
        batch.mask_window = span
        if soft is not None:
            # rows of a block's first step carry a zero signal (the block contributes exactly nothing then)
            states = [mgr.get(r.uid) for r in reqs]
            if all(st.signal is None for st in states):
                batch.canvas_signal = torch.empty((0,), device=eng.device)
            else:
                h = eng.model.self_conditioning_width
                batch.canvas_signal = torch.cat([
                    st.signal if st.signal is not None else torch.zeros((st.length, h), dtype=eng.dtype,
                                                                        device=eng.device) for st in states])
        out = eng.forward_batch(batch, plan, BatchSamplingArgs(), return_logits=True)
        logits = eng.sampler.condition_logits(out.logits, BatchSamplingArgs())
        for i, r in enumerate(reqs):
            st = mgr.get(r.uid)
            st.keep_probs = soft is not None
            st.advance(logits[cu[i]:cu[i + 1]])
            if soft is not None and st.probs is not None:
                st.signal, st.probs = soft(st.probs), None
    sched.stats["steps"] += 1
    sched.stats["decode_tokens"] += total
    sched.stats["denoise_steps"] = sched.stats.get("denoise_steps", 0) + 1


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _ragged_plan(sched, batch: Batch, lens: List[int]):
    """Like ``Scheduler._make_plan(extra_rows=...)`` with a row count per request."""
    from ..engine import StepPlan
    from ..utils import cdiv

    ps, msl = sched.page_size, sched.max_seq_len
    reqs = batch.reqs
    b = len(reqs)
    slots = np.fromiter((r.table_idx for r in reqs), dtype=np.int64, count=b)
    starts = np.fromiter((r.device_len for r in reqs), dtype=np.int64, count=b)
    q_lens = np.asarray(lens, dtype=np.int64)
    ends = starts + q_lens
    for r, end in zip(reqs, ends.tolist()):
        have = sched.alloc_len.get(r.uid, r.cache_handle.cached_len)
        if end > have:
            first, last = cdiv(have, ps), cdiv(end, ps)
            if last > first:
                sched.cache.page_table[r.table_idx, first:last] = sched.cache._take(last - first)
            sched.alloc_len[r.uid] = end
    cu_q = np.zeros(b + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu_q[1:])
    total = int(cu_q[-1])
    row = np.repeat(slots, q_lens)
    pos = np.arange(total, dtype=np.int64) - np.repeat(cu_q[:-1].astype(np.int64), q_lens) + np.repeat(starts, q_lens)
    pages = sched.cache.page_table[row, pos // ps].astype(np.int64)
    max_kv = int(ends.max())
    return StepPlan(token_idx=(row * msl + pos).astype(np.int32), positions=pos.astype(np.int32),
                    out_loc=(pages * ps + pos % ps).astype(np.int32), cu_q=cu_q, seq_lens=ends.astype(np.int32),
                    block_table=np.ascontiguousarray(sched.cache.page_table[slots, : cdiv(max_kv, ps)], dtype=np.int32),
                    sample_rows=np.arange(total, dtype=np.int32), write_idx=np.zeros(0, dtype=np.int32),
                    max_q=int(q_lens.max()), max_kv=max_kv)


def _commit(sched, mgr: CanvasManager, req: Req) -> None:
    """The block is done: emit its candidate tokens, make them committed text (host buffer and token
    pool), reply, and finish the request when it hit an end-of-sequence token or its budget."""
    eng = sched.engine
    st = mgr.get(req.uid)
    tokens = st.emit.to(torch.int32).cpu()
    left = req.sampling_params.max_tokens - req.num_generated
    emitted = tokens[: max(1, min(int(tokens.numel()), left))].tolist()
    hit_eos = False
    if not req.sampling_params.ignore_eos:
        for j, t in enumerate(emitted):
            if t in sched.eos_ids:
                emitted, hit_eos = emitted[: j + 1], True
                break
    n = len(emitted)
    ids = torch.tensor(emitted, dtype=torch.int32)
    req.append_host(ids)
    at = req.table_idx * sched.max_seq_len + req.device_len
    stream_ctx = torch.cuda.stream(eng.stream) if eng.stream is not None else _null()
    with stream_ctx:
        eng.token_pool.view(-1)[at:at + n] = ids.to(eng.device)
    req.device_len += n                            # cached_len stays: these tokens still need causal K/V
    mgr.end(req.uid)
    finished = hit_eos or req.num_generated >= req.sampling_params.max_tokens
    reason = "stop" if hit_eos else ("length" if finished else None)
    replies = []
    for j, t in enumerate(emitted):
        last = j == n - 1
        replies.append(DetokenizeMsg(req.uid, int(t), finished and last, reason if last else None,
                                     prompt_tokens=req.prompt_len, cached_tokens=sched.prefix_len.get(req.uid, 0)))
    sched.stats["blocks"] = sched.stats.get("blocks", 0) + 1
    if finished:
        req.finished, req.finish_reason = True, reason
        mgr.free(req.uid)
        sched.canvas_reqs.pop(req.uid, None)
        sched._free_req_resources(req, insert=True)
    sched.send_result(replies)


def diffusion_loop(sched) -> None:
    mgr: CanvasManager = sched.diffusion
    active: Dict[int, Req] = sched.canvas_reqs
    while not sched._exit:
        for msg in sched.receive_msg(blocking=not (sched.prefill.runnable or active)):
            sched._process_one_msg(msg)
        # requests that were aborted while they held a canvas
        for uid in [u for u, r in active.items() if r.finished]:
            mgr.free(uid)
            active.pop(uid, None)
        # 1. prompts: the ordinary chunked prefill, without a sampled row
        batch, adder = sched.prefill.schedule_next_batch(sched._prefill_budget_now())
        if batch is not None:
            sched._upload_prompts(adder.new_slots)
            for r in batch.reqs:
                sched.reqs[r.uid] = r
                sched.prefix_len.setdefault(r.uid, r.cached_len)
            _encode(sched, batch.reqs)
            for r in batch.reqs:
                if not isinstance(r, ChunkedReq):
                    active[r.uid] = r
        # 2. committed blocks that have no causal K/V yet
        _encode(sched, [r for r in active.values() if r.cached_len < r.device_len])
        # 3. one denoising step for every open canvas (a request without one opens its next block)
        todo = []
        for r in active.values():
            if mgr.get(r.uid) is None:
                room = min(mgr.cfg.block, r.sampling_params.max_tokens - r.num_generated,
                           sched.max_seq_len - r.device_len)
                if room <= 0:
                    continue
                mgr.begin(r.uid, room, r.sampling_params.seed)
            todo.append(r)
        todo.sort(key=lambda r: r.uid)
        if todo:
            _denoise(sched, mgr, todo)
            for r in todo:
                if mgr.get(r.uid).finished:
                    _commit(sched, mgr, r)
        sched._after_iteration()
