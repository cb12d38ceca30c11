"""Per-rank scheduler: admits requests, packs prefill chunks and decode batches, drives the
engine, commits sampled tokens and replies.

Loop structure follows python/minisgl/scheduler/scheduler.py (:1101 overlap loop, :1161
normal loop, :1458 result processing, :1596 message handling, :1647 resource release):

* ``overlap_loop``: while the GPU runs step *n* the host receives messages, plans step
  *n+1* and launches it, and only then blocks on the tokens of step *n*. Length bookkeeping
  (``complete_one``) happens at launch time because it does not depend on token values; the
  sampled ids reach the next step through the device-resident token pool.
* ``normal_loop``: the synchronous variant (one step fully processed before the next).

Speculative decoding and expert-parallel lockstep are mixed in from ``spec_step.py`` and
``ep.py``.
"""
from __future__ import annotations

import contextlib

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..config import SchedulerConfig
from ..core import Batch, ChunkedReq, Req, SamplingParams
from ..engine import BatchSamplingArgs, Engine, ForwardOutput, StepPlan
from ..env import ENV
from ..message import AbortBackendMsg, BaseMsg, BatchMsg, DetokenizeMsg, ExitMsg, StatsMsg, UserMsg
from ..utils import cdiv, init_logger
from .cache import CacheManager
from .decode import DecodeManager
from .prefill import PrefillManager
from .table import TableManager

logger = init_logger(__name__)


@dataclass
class Ongoing:
    batch: Batch
    sampled: List[Req]
    output: ForwardOutput
    launched_at: float


class RequestAllFinished(Exception):
    """Raised by an offline receive hook when no work is left."""


class Scheduler:
    def __init__(self, config: SchedulerConfig, engine: Optional[Engine] = None) -> None:
        self.config = config
        self.engine = engine if engine is not None else Engine(config)
        eng = self.engine
        self.page_size = eng.page_size
        self.table = TableManager(config.max_running_req)
        # A recurrent state cannot be rewound to a matched prefix: hybrid models reuse a cached prefix
        # only up to a boundary at which a snapshot of the state was taken (the snapshot radix cache),
        # or admit every request with an empty prefix when snapshots are off
        # (python/minisgl/engine/config.py:75-133).
        cache_type = config.cache_type
        self._snap_pending: Dict[int, List] = {}
        self._snap_ids = 0
        self._snapshots_on = False
        # what keeps and restores per-request state at a prefix boundary: the recurrent-state cache, or the
        # sliding-window pool (its window pages below the boundary); same interface
        self._keeper = eng.gdn_state if eng.gdn_state is not None else eng.swa
        if eng.model_config.is_recurrent or eng.swa is not None:
            self._snapshots_on = (cache_type == "radix" and ENV.RECURRENT_SNAPSHOT_MIB.value > 0
                                  and self._keeper is not None)
            cache_type = "radix_snapshot" if self._snapshots_on else "naive"
        if eng.model_config.is_recurrent and config.spec_algorithm != "none" and getattr(
                config, "spec_tree_width", 1) > 1:
            # siblings of a draft tree would each need their own copy of the running state
            raise ValueError("tree verification is not available for models with recurrent layers; "
                             "use a draft chain (spec tree width 1)")
        self.cache = CacheManager(eng.num_pages, eng.page_size, eng.num_slots, eng.max_pages_per_seq,
                                  cache_type)
        if self._snapshots_on:
            pc = self.cache.prefix_cache
            pc.capacity = max(4, (ENV.RECURRENT_SNAPSHOT_MIB.value << 20) // max(self._keeper.slot_nbytes(), 1))
            host_mib = ENV.RECURRENT_SNAPSHOT_HOST_MIB.value
            if host_mib > 0 and eng.gdn_state is not None:
                # snapshots in page-locked host frames: the prefix cache may keep what is left after the
                # frames that running requests hold for boundaries not attached to the tree yet
                frames = eng.gdn_state.attach_host_arena(host_mib << 20)
                if frames > 0:
                    pc.capacity = max(4, frames - min(frames // 2, 6 * config.max_running_req))
            pc.on_drop = self._keeper.drop_snapshot
            every = max(ENV.RECURRENT_SNAPSHOT_TOKENS.value, eng.page_size)
            self._snap_every = (every + eng.page_size - 1) // eng.page_size * eng.page_size
            logger.info_rank0("prefix-boundary state kept every %d tokens and at chunk ends, up to %d at a time (%.1f MiB each)",
                              self._snap_every, pc.capacity, self._keeper.slot_nbytes() / 2 ** 20)
        self.decode = DecodeManager(eng.page_size)
        self.prefill = PrefillManager(self.cache, self.table, self.decode)
        self.max_seq_len = eng.max_seq_len
        self.eos_ids = set(eng.model_config.eos_token_ids)
        self.reqs: Dict[int, Req] = {}
        self.alloc_len: Dict[int, int] = {}      # uid -> token positions that own a KV slot
        self.prefix_len: Dict[int, int] = {}     # uid -> cached tokens at admission (reporting)
        self.finished_uids: set = set()
        self.mm: Dict[int, tuple] = {}          # uid -> (placeholder positions, image features) of multimodal requests
        self.last_state_digests: Dict[int, dict] = {}   # uid -> digests of its last prefill step (MSGL_STATE_DIGEST)
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "steps": 0, "finished": 0,
                      "spec_drafted": 0, "spec_accepted": 0, "spec_emitted": 0, "spec_steps": 0}
        self._exit = False
        self._last_stats_flush = time.monotonic()
        from ..utils.tracing import HostStages, StepProfiler

        self._step_profiler = StepProfiler(getattr(config, "tp_rank", 0))
        self._host_stages = HostStages()
        self._dummy_slot = eng.num_slots - 1
        self._use_overlap = not (config.disable_overlap or ENV.DISABLE_OVERLAP.value) and eng.device.type == "cuda"
        # block-diffusion models run a loop of their own (scheduler/diffusion.py)
        from .diffusion import make_canvas_manager

        self.diffusion = make_canvas_manager(self)
        self.canvas_reqs: Dict[int, Req] = {}
        self.proposer = None
        if config.spec_algorithm != "none":
            from ..spec import make_proposer

            self.proposer = make_proposer(config, self)
            self._use_overlap = False
            from .spec_step import device_runner

            device_runner(self)   # GPU engines: build the on-device step and capture its graphs at boot

    # ------------------------------------------------------------------ I/O hooks
    def receive_msg(self, blocking: bool) -> List[BaseMsg]:
        raise NotImplementedError

    def send_result(self, replies: List[DetokenizeMsg]) -> None:
        raise NotImplementedError

    # ------------------------------------------------------------------ messages
    def _process_one_msg(self, msg: BaseMsg) -> None:
        if isinstance(msg, BatchMsg):
            for m in msg.data:
                self._process_one_msg(m)
        elif isinstance(msg, ExitMsg):
            self._exit = True
        elif isinstance(msg, UserMsg):
            self._admit(msg)
        elif isinstance(msg, AbortBackendMsg):
            self._abort(msg.uid)
        else:
            logger.warning("ignoring unknown message %r", type(msg).__name__)

    def _admit(self, msg: UserMsg) -> None:
        ids = msg.input_ids.to(torch.int32).reshape(-1)
        n = int(ids.numel())
        params = msg.sampling_params
        # an over-long prompt is answered with an error, it never crashes the rank
        # (python/minisgl/scheduler/scheduler.py:1616-1630)
        if n == 0 or n >= self.max_seq_len:
            self.send_result([DetokenizeMsg(msg.uid, 0, True, "error",
                                            error=f"prompt of {n} tokens exceeds the limit {self.max_seq_len - 1}")])
            return
        max_new = min(params.max_tokens, self.max_seq_len - n)
        if max_new != params.max_tokens:
            import dataclasses as _dc

            params = _dc.replace(params, max_tokens=max_new)
        need_pages = cdiv(n + max_new, self.page_size)
        if need_pages > self.cache.num_pages:
            self.send_result([DetokenizeMsg(msg.uid, 0, True, "error",
                                            error="request does not fit in the KV cache")])
            return
        if getattr(msg, "images", None) is not None:
            ids = self._admit_images(msg.uid, ids, msg.images)
            if ids is None:
                return
        self.prefill.add_one_req(msg.uid, ids, params)
        if msg.uid in self.mm:
            self.prefill.pending[-1].spans = self.mm[msg.uid][2]      # a prefill chunk must not cut an image
        from ..utils.tracing import log_request

        log_request("admit", msg.uid, prompt=n, max_new=max_new)

    def _admit_images(self, uid: int, ids: torch.Tensor, images: torch.Tensor) -> Optional[torch.Tensor]:
        """Run the vision tower over a request's images (``[n, 3, S, S]`` uint8) and remember the
        projected features for the placeholder positions of its prompt. The placeholder ids are
        replaced by ids outside the vocabulary derived from the image content: the embedding of
        such an id is zero (it is overwritten by the image feature) and the prefix cache tells two
        images apart (python/minisgl/tokenizer/vision.py:92 expands the placeholders; the reference
        runs its tower in the model's forward)."""
        import hashlib

        eng = self.engine
        tower = eng.vision
        if tower is None:
            self.send_result([DetokenizeMsg(uid, 0, True, "error", error="this model takes no image input")])
            return None
        vc = tower.cfg
        per = vc.tokens_per_image
        pos = (ids == vc.image_token_id).nonzero().flatten()
        n = int(images.shape[0])
        if int(pos.numel()) != n * per or tuple(images.shape[1:]) != (3, vc.image_size, vc.image_size):
            self.send_result([DetokenizeMsg(uid, 0, True, "error", error=(
                f"{n} image(s) of shape {tuple(images.shape[1:])} against {int(pos.numel())} placeholder tokens "
                f"({per} per {vc.image_size}x{vc.image_size} image expected)"))])
            return None
        ctx = torch.cuda.stream(eng.stream) if eng.stream is not None else contextlib.nullcontext()
        with ctx:
            px = images.to(eng.device, non_blocking=True).to(torch.float32) / 255.0
            emb = tower.image_embeddings((px - 0.5) / 0.5)
        ids = ids.clone()
        vocab = eng.model_config.vocab_size
        for i in range(n):
            h = int.from_bytes(hashlib.sha1(images[i].contiguous().numpy().tobytes()).digest()[:4], "little")
            ids[pos[i * per:(i + 1) * per]] = (vocab + h % (1 << 29) + torch.arange(per)).to(ids.dtype)
        where = pos.numpy().astype(np.int64)
        spans = np.stack([where[0::per], where[per - 1::per] + 1], axis=1) if n else np.zeros((0, 2), dtype=np.int64)
        self.mm[uid] = (where, emb, spans)
        return ids

    def _image_rows(self, batch: Batch, plan: StepPlan) -> None:
        """Rows of a prefill step that are image placeholders, and the features that go there."""
        rows, vals = [], []
        for i, r in enumerate(batch.reqs):
            entry = self.mm.get(r.uid)
            if entry is None:
                continue
            pos, emb, _spans = entry
            lo, hi = int(r.cached_len), int(r.device_len)
            sel = np.nonzero((pos >= lo) & (pos < hi))[0]
            if sel.size:
                rows.append(int(plan.cu_q[i]) + (pos[sel] - lo))
                vals.append(emb[torch.as_tensor(sel, device=emb.device)])
        if rows:
            batch.mm_rows = torch.as_tensor(np.concatenate(rows), dtype=torch.int64).to(self.engine.device)
            batch.mm_values = torch.cat(vals)
            if ENV.IMAGE_BIDIRECTIONAL.value and self.engine.model_config.image_bidirectional:
                self._image_masks(batch, plan)

    def _image_masks(self, batch: Batch, plan: StepPlan) -> None:
        """Additive masks of a prefill step that computes image rows: causal everywhere, and the tokens of
        one image see each other in both directions (the published Gemma-3 prefill). A mask replaces the
        kernel's causal and window rules for every row of the step, so both are written out here, and the
        sliding-window layers get a mask of their own with their window in it."""
        mc = self.engine.model_config
        window = int(mc.sliding_window) if (mc.sliding_window and mc.swa_layers) else 0
        total, max_kv = plan.num_tokens, int(plan.max_kv)
        neg = float("-inf")
        full = torch.full((total, max_kv), neg, dtype=torch.float32)
        local = torch.full((total, max_kv), neg, dtype=torch.float32) if window else None
        k = torch.arange(max_kv)[None, :]
        for i, r in enumerate(batch.reqs):
            lo, hi = int(r.cached_len), int(r.device_len)
            q = torch.arange(lo, hi)[:, None]
            seen = (k <= q)
            same = torch.zeros_like(seen)
            entry = self.mm.get(r.uid)
            if entry is not None:
                image_of = torch.full((max(hi, 1),), -1, dtype=torch.int64)
                for j, (a, b) in enumerate(entry[2].tolist()):
                    image_of[a:min(b, hi)] = j
                iq = image_of[lo:hi][:, None]
                ik = torch.full((max_kv,), -2, dtype=torch.int64)
                ik[:hi] = image_of[:hi]
                same = (iq == ik[None, :]) & (iq >= 0)
            rows = slice(int(plan.cu_q[i]), int(plan.cu_q[i + 1]))
            inside = k < hi
            full[rows] = torch.where((seen | same) & inside, 0.0, neg)
            if local is not None:
                local[rows] = torch.where(((seen & (k > q - window)) | same) & inside, 0.0, neg)
        dev = self.engine.device
        batch.tree_mask = full.to(dev)
        batch.tree_mask_swa = local.to(dev) if local is not None else None

    def _abort(self, uid: int) -> None:
        pending = self.prefill.abort(uid)
        if pending is not None:
            self.mm.pop(uid, None)
        if pending is not None:
            if pending.chunked is not None:
                self._free_req_resources(pending.chunked, insert=False)
            return
        req = self.reqs.get(uid)
        if req is not None and not req.finished:
            req.finished = True
            req.finish_reason = "abort"
            self._free_req_resources(req, insert=True)

    # ------------------------------------------------------------------ planning
    def _free_device_bytes(self) -> Optional[int]:
        """Device memory a forward can still take: what the driver reports free plus the caching
        allocator's reserved-but-unallocated blocks (at steady state that cache is most of the headroom)."""
        if self.engine.device.type != "cuda":
            return None
        try:
            free, _total = torch.cuda.mem_get_info(self.engine.device)
            return int(free + torch.cuda.memory_reserved(self.engine.device)
                       - torch.cuda.memory_allocated(self.engine.device))
        except Exception:      # the guard must never break scheduling
            return None

    def _prefill_budget_now(self) -> int:
        """Prefill tokens this step may take: the configured chunk, shrunk when free device memory
        cannot hold that chunk's activations (python/minisgl/scheduler/scheduler.py:2524-2570). The
        peak of a prefill step is proportional to its tokens, not to the context behind them, so the
        largest safe step is ``(free - safety) / bytes per token``; the step shrinks in whole pages
        and never below 1024 tokens (a step too small to make progress is worse than a failed one)."""
        base = self.config.max_extend_tokens
        if not self.prefill.runnable:                  # nothing to prefill: skip the driver query
            return base
        free = self._free_device_bytes()
        if free is None:
            return base
        mc, tp = self.engine.model_config, max(self.config.tp_size, 1)
        widest = max(2 * mc.intermediate_size // tp, mc.q_size + 2 * mc.kv_size, mc.hidden_size * 4)
        per_token = widest * 2 * 4                       # the engine's sizing rule for a chunk's intermediates
        affordable = (free - (1 << 30)) // max(per_token, 1)
        if affordable >= base:
            return base
        page = max(1, self.page_size)
        budget = max(min(base, max(page, 1024)), (int(affordable) // page) * page)
        self._act_guard_trips = getattr(self, "_act_guard_trips", 0) + 1
        if self._act_guard_trips <= 3 or self._act_guard_trips % 100 == 0:
            logger.warning("prefill activation guard: %.2f GiB free affords %d tokens at %d KiB/token: step of %d "
                           "instead of %d", free / 2 ** 30, affordable, per_token // 1024, budget, base)
        return budget

    def _schedule_next_batch(self) -> Optional[Batch]:
        batch, adder = self.prefill.schedule_next_batch(self._prefill_budget_now())
        if batch is not None:
            self._upload_prompts(adder.new_slots)
            if adder.restores:
                self._restore_states(adder.restores)
            for req in batch.reqs:
                self.reqs[req.uid] = req
                self.prefix_len.setdefault(req.uid, req.cached_len)
            return batch
        return self.decode.schedule_next_batch()

    def _upload_prompts(self, new_slots) -> None:
        """Copy newly admitted prompts from pinned host memory into the token pool, on the
        engine's stream so the copy is ordered before the forward that reads it."""
        pool = self.engine.token_pool
        if not new_slots:
            return
        if pool.is_cuda:
            with torch.cuda.stream(self.engine.stream):
                for slot, ids, _cached in new_slots:
                    pool[slot, : ids.numel()].copy_(ids.pin_memory(), non_blocking=True)
                    self.engine.h2d_bytes += 4 * int(ids.numel())
        else:
            for slot, ids, _cached in new_slots:
                pool[slot, : ids.numel()].copy_(ids)

    def _restore_states(self, restores) -> None:
        """Prefix hits of a recurrent model: copy the snapshot of each matched boundary into the
        request's state slot, on the engine's stream ahead of the forward that continues from it."""
        st = self._keeper
        if self.engine.device.type == "cuda":
            with torch.cuda.stream(self.engine.stream):
                for slot, key in restores:
                    st.restore(slot, key)
        else:
            for slot, key in restores:
                st.restore(slot, key)

    def _snapshot_states(self, batch: Batch, ends) -> None:
        """After a step was launched: keep the recurrent state of every request that has just reached
        a reusable boundary (a page multiple at the end of a prefill chunk, or every
        ``MSGL_RECURRENT_SNAPSHOT_TOKENS`` tokens). The copies are ordered behind the step on the
        engine's stream; the ids are attached to the prefix cache when the request finishes."""
        st = self._keeper
        todo = []
        for r, end in zip(batch.reqs, ends):
            if end % self.page_size:
                continue
            if isinstance(r, ChunkedReq) or end % self._snap_every == 0:
                todo.append((r, int(end)))
        if not todo:
            return

        def take():
            for r, end in todo:
                self._snap_ids += 1
                st.snapshot(r.table_idx, self._snap_ids, host=False, end=end)
                pend = self._snap_pending.setdefault(r.uid, [])
                pend.append((end, self._snap_ids))
                if len(pend) > 6:                      # keep the earliest (shared prompts) and the latest
                    _, old = pend.pop(3)
                    st.drop_snapshot(old)

        if self.engine.device.type == "cuda":
            with torch.cuda.stream(self.engine.stream):
                take()
        else:
            take()

    def _make_plan(self, batch: Batch, extra_rows: int = 0) -> StepPlan:
        """Allocate pages and build the step's index arrays. ``extra_rows`` > 0 plans a
        verify step: every request feeds ``1 + extra_rows`` tokens."""
        ps = self.page_size
        msl = self.max_seq_len
        reqs = batch.reqs
        b = len(reqs)
        slots = np.fromiter((r.table_idx for r in reqs), dtype=np.int64, count=b)
        starts = np.fromiter((r.cached_len for r in reqs), dtype=np.int64, count=b)
        ends = np.fromiter((r.device_len for r in reqs), dtype=np.int64, count=b) + extra_rows
        for r, end in zip(reqs, ends.tolist()):
            have = self.alloc_len.get(r.uid, r.cache_handle.cached_len)
            if end > have:
                first, last = cdiv(have, ps), cdiv(end, ps)
                if last > first:
                    self.cache.page_table[r.table_idx, first:last] = self.cache._take(last - first)
                self.alloc_len[r.uid] = end
        swa = self.engine.swa
        if swa is not None:
            # sliding-window pool: pages that left the window of this step's first query go back before
            # this step's new pages are taken (earlier steps that read them are ahead on the stream)
            for r, start, end in zip(reqs, starts.tolist(), ends.tolist()):
                swa.trim(r.table_idx, start)
                swa.ensure(r.table_idx, end)
        q_lens = ends - starts
        cu_q = np.zeros(b + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu_q[1:])
        total = int(cu_q[-1])
        if int(q_lens.max()) == 1:
            pos = starts
            row = slots
        else:
            row = np.repeat(slots, q_lens)
            pos = np.arange(total, dtype=np.int64) - np.repeat(cu_q[:-1].astype(np.int64), q_lens) + np.repeat(starts, q_lens)
        token_idx = (row * msl + pos).astype(np.int32)
        pages = self.cache.page_table[row, pos // ps].astype(np.int64)
        out_loc = (pages * ps + pos % ps).astype(np.int32)
        max_kv = int(ends.max())
        n_pages = cdiv(max_kv, ps)
        block_table = self.cache.page_table[slots, :n_pages]
        if batch.spec_verify:
            sample_rows = np.arange(total, dtype=np.int32)
            write_idx = np.zeros(0, dtype=np.int32)
        else:
            keep = np.fromiter((not isinstance(r, ChunkedReq) for r in reqs), dtype=bool, count=b)
            sample_rows = (cu_q[1:] - 1)[keep].astype(np.int32)
            write_idx = (slots * msl + ends)[keep].astype(np.int32)
        return StepPlan(
            token_idx=token_idx, positions=pos.astype(np.int32), out_loc=out_loc, cu_q=cu_q,
            seq_lens=ends.astype(np.int32), block_table=np.ascontiguousarray(block_table, dtype=np.int32),
            sample_rows=sample_rows, write_idx=write_idx, max_q=int(q_lens.max()), max_kv=max_kv,
        )

    # ------------------------------------------------------------------ forward
    def _forward(self, batch: Batch) -> Ongoing:
        plan = self._make_plan(batch)
        if self.mm and batch.is_prefill:
            self._image_rows(batch, plan)
        capture = getattr(self.proposer, "capture_layers", None)
        if capture:
            batch.capture_layers = list(capture)
            self._feature_meta = (plan.cu_q.copy(), [r.cached_len for r in batch.reqs])
        sampled = [r for r in batch.reqs if not isinstance(r, ChunkedReq)]
        args = self.engine.sampler.prepare(sampled) if sampled else BatchSamplingArgs()
        self._attach_constraints(sampled, args)
        out = self.engine.forward_batch(batch, plan, args)
        if self._snapshots_on:
            self._snapshot_states(batch, plan.seq_lens.tolist())
        digest = batch.is_prefill and ENV.STATE_DIGEST.value
        n_tok = plan.num_tokens
        if batch.is_prefill:
            self.stats["prefill_tokens"] += n_tok
        else:
            self.stats["decode_tokens"] += n_tok
        self.stats["steps"] += 1
        # length bookkeeping does not need token values
        for r in batch.reqs:
            if isinstance(r, ChunkedReq):
                r.cached_len = r.device_len
            else:
                r.complete_one()
        if digest:
            from ..kvcache import state_digest

            for r in batch.reqs:        # lengths have just moved: cached_len covers what this step computed
                state_digest.log_request(self, r, "chunk" if isinstance(r, ChunkedReq) else "prefill")
        if batch.is_prefill:
            self.decode.add_reqs(sampled)
        self.decode.filter_finished()
        return Ongoing(batch, sampled, out, time.monotonic())

    # ------------------------------------------------------------------ constrained decoding
    def _constraint_state(self):
        """Lazily built grammar backend, tokenizer and per-request gates."""
        st = getattr(self, "_cstate", None)
        if st is None:
            from ..engine.grammar import GrammarBackend, GrammarState
            from ..tokenizer.simple import load_tokenizer

            tok = load_tokenizer(self.config.model_path)
            backend = GrammarBackend(tok, vocab_size=self.engine.model_config.vocab_size,
                                     stop_token_ids=sorted(self.eos_ids) or None)
            st = self._cstate = {"tok": tok, "grammar": GrammarState(backend), "think": {}, "tool": {}}
        return st

    def _needs_constraints(self, req: Req) -> bool:
        sp = req.sampling_params
        return sp.grammar is not None or bool(sp.tool_call_closers) or (sp.think_close_delim is not None and sp.think_budget > 0)

    def _gates_for(self, req: Req):
        from .think_gate import ThinkGate, ToolCallGate

        st = self._constraint_state()
        sp = req.sampling_params
        enc = lambda text: list(st["tok"].encode(text))
        think = st["think"].get(req.uid)
        if think is None and sp.think_close_delim is not None:
            # a direct answer (the model's own answer-turn header) and a closer that names a recipient
            # in its middle (prefix .. up to 16 arbitrary tokens .. suffix) release the gate as well
            answers = [enc(sp.think_answer_delim)] if sp.think_answer_delim else []
            wild = []
            if sp.think_close_prefix and sp.think_close_suffix:
                wild.append((tuple(enc(sp.think_close_prefix)), tuple(enc(sp.think_close_suffix)), 16))
            think = st["think"][req.uid] = ThinkGate(
                enc(sp.think_close_delim), [enc(t) for t in sp.think_tool_release], sp.think_budget,
                span_open=sp.think_span_open or sp.think_budget > 0, answer_patterns=answers, close_wildcards=wild,
                loop_period=ENV.THINK_LOOP_PERIOD.value, loop_span=ENV.THINK_LOOP_SPAN.value,
                loop_reps=ENV.THINK_LOOP_REPS.value)
        tool = st["tool"].get(req.uid)
        if tool is None and sp.tool_call_openers and sp.tool_call_closers:
            tool = st["tool"][req.uid] = ToolCallGate([enc(t) for t in sp.tool_call_openers],
                                                      [enc(t) for t in sp.tool_call_closers],
                                                      limit=ENV.TOOLCALL_RUNAWAY_LIMIT.value)
        return think, tool

    def _attach_constraints(self, reqs: Sequence[Req], args: BatchSamplingArgs) -> None:
        """Build the allowed-token bitmask of this step: grammar masks (once a reasoning span
        is over), a single forced token when a reasoning budget ran out, and end-of-sequence
        suppression while a tool call is open (python/minisgl/scheduler/scheduler.py:2343)."""
        rows = [i for i, r in enumerate(reqs) if self._needs_constraints(r)]
        if not rows:
            return
        st = self._constraint_state()
        gs = st["grammar"]
        backend = gs.backend
        bm = backend.allocate_bitmask(len(rows))
        bm.fill_(-1)
        for j, i in enumerate(rows):
            r = reqs[i]
            sp = r.sampling_params
            think, tool = self._gates_for(r)
            forced = think.forced_token() if think is not None else None
            if forced is not None:
                bm[j].zero_()
                bm[j, forced // 32] = 1 << (forced % 32) if forced % 32 != 31 else -(1 << 31)
                continue
            if sp.grammar is not None and (think is None or think.grammar_active):
                backend.fill(gs.ensure(r.uid, sp.grammar), bm, j)
            # no end of turn inside an open tool call, nor inside a reasoning span that the prompt
            # opened and whose budget will force the close delimiter out (a thinking model that stops there returns
            # a blank answer; python/minisgl/engine/sample.py:29-32)
            thinking = think is not None and not think.released and think.budget > 0 and sp.think_span_open
            if (tool is not None and tool.suppress_eos) or thinking:
                for e in self.eos_ids:
                    word, bit = e // 32, e % 32
                    mask = ~(1 << bit) if bit != 31 else 0x7FFFFFFF
                    bm[j, word] = int(bm[j, word]) & mask
        args.bitmask = bm.to(self.engine.device, non_blocking=True)
        args.bitmask_rows = torch.tensor(rows, dtype=torch.int64, device=self.engine.device)

    def _observe_token(self, req: Req, tok: int) -> None:
        st = getattr(self, "_cstate", None)
        if st is None or not self._needs_constraints(req):
            return
        think, tool = st["think"].get(req.uid), st["tool"].get(req.uid)
        active = think is None or think.grammar_active
        if think is not None:
            think.observe(tok)
            period = think.take_loop_report()
            if period:
                logger.warning("request %d repeats a block of %d token(s) inside its reasoning span: closing the span",
                               req.uid, period)
        if tool is not None:
            tool.observe(tok)
        if req.sampling_params.grammar is not None and active:
            st["grammar"].accept(req.uid, tok)

    def _tool_call_runaway(self, req: Req) -> bool:
        """A tool call that has run past ``MSGL_TOOLCALL_RUNAWAY_LIMIT`` tokens without closing ends
        the request (python/minisgl/scheduler/think_gate.py:123-230: EOS is masked inside a call, so
        a degenerate model would otherwise run to the token cap)."""
        st = getattr(self, "_cstate", None)
        tool = st["tool"].get(req.uid) if st is not None else None
        if tool is not None and tool.runaway:
            logger.warning("request %d: tool call still open after %d tokens, ending the request", req.uid, tool.inside)
            return True
        return False

    def _forget_constraints(self, uid: int) -> None:
        st = getattr(self, "_cstate", None)
        if st is not None:
            st["grammar"].finish(uid)
            st["think"].pop(uid, None)
            st["tool"].pop(uid, None)

    # ------------------------------------------------------------------ results
    def _process_last_data(self, ongoing: Optional[Ongoing]) -> None:
        if ongoing is None:
            return
        tokens = ongoing.output.wait()
        self._check_comm_health()
        sample = ongoing.output.sample
        lp = sample.logprobs.tolist() if sample is not None and sample.logprobs is not None else None
        tlp = tids = None
        if sample is not None and sample.top_logprobs is not None:
            tlp, tids = sample.top_logprobs.tolist(), sample.top_ids.tolist()
        replies: List[DetokenizeMsg] = []
        toks = tokens.tolist()
        for i, req in enumerate(ongoing.sampled):
            if req.finished:
                continue  # finished or aborted while this step was in flight
            tok = int(toks[i])
            req.append_host(tokens[i : i + 1])
            self._observe_token(req, tok)
            reason = None
            if not req.sampling_params.ignore_eos and tok in self.eos_ids:
                reason = "stop"
            elif req.num_generated >= req.sampling_params.max_tokens:
                reason = "length"
            elif self._tool_call_runaway(req):
                reason = "length"
            msg = DetokenizeMsg(req.uid, tok, reason is not None, reason,
                                prompt_tokens=req.prompt_len, cached_tokens=self.prefix_len.get(req.uid, 0))
            if lp is not None and req.sampling_params.logprobs > 0:
                msg.logprob = lp[i]
                n = req.sampling_params.logprobs
                msg.top_logprobs = [[tids[i][j], tlp[i][j]] for j in range(n)]
            replies.append(msg)
            if reason is not None:
                req.finished = True
                req.finish_reason = reason
                self._free_req_resources(req, insert=True)
        if replies:
            self.send_result(replies)

    def _check_comm_health(self) -> None:
        """Every ``MSGL_COMM_HEALTH_STEPS`` steps (the host has just synchronised with the device
        anyway) the ranks of the tensor-parallel group agree, over the CPU group, on the worst
        status word of the peer-memory collectives. A wait that ran out on any rank means a peer
        is missing or slow: every rank leaves the fused path on this same step, decode leaves its
        captured graphs (which contain the fused kernels) for eager steps on the NCCL path, and the
        requests that were running are ended with an error, because steps since the last clean
        check may have summed incomplete partials. A peer that is really gone is then caught by
        the process-group timeout and the crash watchdog."""
        every = max(1, ENV.COMM_HEALTH_STEPS.value)
        if self.config.tp_size == 1 or self.stats["steps"] % every != 0:
            return
        from ..parallel.comm import get_comm

        for impl in get_comm().impls:
            check = getattr(impl, "check_health", None)
            if check is not None and getattr(impl, "healthy", True) and not check():
                logger.warning("peer-memory collectives disabled after a device-side timeout")
                self.engine.graph_runner = None
                self._fail_running("a collective timed out; the request was ended because its state may be incomplete")

    def _fail_running(self, why: str) -> None:
        replies = []
        for req in list(self.decode.running.values()):
            if req.finished:
                continue
            req.finished, req.finish_reason = True, "error"
            replies.append(DetokenizeMsg(req.uid, 0, True, "error", error=why))
            self._free_req_resources(req, insert=False)
        self.decode.filter_finished()
        if replies:
            self.send_result(replies)

    def _free_req_resources(self, req: Req, insert: bool) -> None:
        if req.resources_freed:  # several paths can reach a request; free exactly once
            return
        req.resources_freed = True
        self.decode.remove(req)
        self.mm.pop(req.uid, None)
        if self.engine.swa is not None:
            self.engine.swa.release(req.table_idx)
        alloc = self.alloc_len.pop(req.uid, req.cache_handle.cached_len)
        # KV is valid for tokens that were both fed and known on the host
        req.cached_len = min(req.cached_len, int(req.input_ids.numel()))
        unused = self.cache.finish_req(req, alloc, insert=insert, snapshots=self._snap_pending.pop(req.uid, None))
        for key in unused or ():
            self._keeper.drop_snapshot(key)
        self.table.free(req.table_idx)
        self._forget_constraints(req.uid)
        self.reqs.pop(req.uid, None)
        self.prefix_len.pop(req.uid, None)
        self.stats["finished"] += 1
        from ..utils.tracing import log_request

        log_request("finish", req.uid, tokens=int(req.device_len))

    # ------------------------------------------------------------------ loops
    @property
    def has_work(self) -> bool:
        return self.prefill.runnable or self.decode.runnable

    def overlap_loop(self) -> None:
        last: Optional[Ongoing] = None
        hp = self._host_stages
        while not self._exit:
            blocking = not self.has_work and last is None
            with hp.stage("receive"):
                for msg in self.receive_msg(blocking):
                    self._process_one_msg(msg)
            if last is not None and any(self._needs_constraints(r) for r in last.sampled):
                # a grammar mask depends on the token of the step in flight: no overlap for this iteration
                self._process_last_data(last)
                last = None
            with hp.stage("schedule"):
                batch = self._schedule_next_batch()
            with hp.stage("plan+launch"):
                ongoing = self._forward(batch) if batch is not None else None
            with hp.stage("results"):
                self._process_last_data(last)
            last = ongoing
            self._after_iteration()
        self._process_last_data(last)

    def normal_loop(self) -> None:
        hp = self._host_stages
        while not self._exit:
            with hp.stage("receive"):
                for msg in self.receive_msg(blocking=not self.has_work):
                    self._process_one_msg(msg)
            if self.proposer is not None and not self.prefill.runnable and self.decode.runnable:
                with hp.stage("spec_step"):
                    self._spec_decode_step()
            else:
                with hp.stage("schedule"):
                    batch = self._schedule_next_batch()
                if batch is not None:
                    with hp.stage("plan+launch"):
                        ongoing = self._forward(batch)
                    with hp.stage("results"):
                        self._process_last_data(ongoing)
                    if self.proposer is not None and batch.is_prefill:
                        self._feed_prefill_features(batch)
                        self.proposer.on_prefill(ongoing.sampled)
            self._after_iteration()

    def _after_iteration(self) -> None:
        self._step_profiler.on_step(self.stats["steps"])
        self._host_stages.tick()
        self._maybe_exit_after_steps()

    def _maybe_exit_after_steps(self) -> None:
        limit = ENV.EXIT_AFTER_STEPS.value
        if limit and self.stats["steps"] >= limit:
            self._exit = True

    def run_forever(self) -> None:
        try:
            self._run_loops()
        finally:
            self._step_profiler.close()
            if self._host_stages.enabled:
                logger.info("hostprof %s", self._host_stages.summary())
            gt = getattr(self.engine.graph_runner, "timer", None) if self.engine is not None else None
            if gt is not None and gt.enabled:
                logger.info("graph replay timing: %s", gt.summary())

    def _run_loops(self) -> None:
        try:
            if self.config.enable_ep and self.config.dp_size > 1:
                from .ep import ep_lockstep_loop

                ep_lockstep_loop(self)
            elif self.diffusion is not None:
                from .diffusion import diffusion_loop

                diffusion_loop(self)
            elif self._use_overlap:
                self.overlap_loop()
            else:
                self.normal_loop()
        except RequestAllFinished:
            pass
        finally:
            self._flush_ghost_oracle()

    def _flush_ghost_oracle(self) -> None:
        """Log the prefix-reuse oracle's counters and persist them when a directory is configured."""
        ghost = getattr(getattr(self, "cache", None), "ghost", None)
        if ghost is None or ghost.requests == 0:
            return
        from ..kvcache.ghost_oracle import oracle_path

        logger.info("%s", ghost.report())
        path = oracle_path(self.config.model_path, self.config.dp_rank)
        if path:
            try:
                ghost.save(path)
            except OSError as exc:
                logger.warning("ghost oracle state not saved: %s", exc)

    # ------------------------------------------------------------------ spec decode
    def _feed_prefill_features(self, batch: Batch) -> None:
        """Hand the target's auxiliary hidden states of a prefill step to a feature-based
        proposer (EAGLE3 / MTP). Row i of a request pairs the feature of position i with the token
        at position i+1; the last row of a partially prefilled prompt waits for the next chunk."""
        prop = self.proposer
        aux = self.engine.ctx.aux_hidden
        if not hasattr(prop, "on_features") or not aux:
            return
        from .spec_step import _engine_stream, device_runner

        runner = device_runner(self)
        if runner is not None and runner.draft is not None:
            # batched draft update on the device: same rows, positions and K/V slots as the step
            slots = np.fromiter((r.table_idx for r in batch.reqs), dtype=np.int64, count=len(batch.reqs))
            with _engine_stream(self.engine):
                runner.feed_prefill(batch, batch.token_idx, slots, batch.host_cu_q)
            return
        cu, starts = self._feature_meta
        carry = getattr(self, "_feature_carry", None)
        if carry is None:
            carry = self._feature_carry = {}
        for i, req in enumerate(batch.reqs):
            rows = [a[cu[i]:cu[i + 1]] for a in aux]
            first = starts[i]
            prev = carry.pop(req.uid, None)
            if prev is not None:
                rows = [torch.cat([p, r]) for p, r in zip(prev, rows)]
                first -= 1
            n = rows[0].shape[0]
            ids = req.input_ids  # after the step: prompt (+ the sampled token for a finished prefill)
            avail = int(ids.numel()) - (first + 1)   # tokens known at positions first+1 ...
            use = min(n, avail)
            if use < n:
                carry[req.uid] = [r[use:] for r in rows]
            if use > 0:
                prop.on_features(req, [r[:use] for r in rows], first, ids[first + 1:first + 1 + use])
        self.engine.ctx.aux_hidden = None

    def _spec_decode_step(self) -> None:
        from .spec_step import spec_decode_step

        spec_decode_step(self)

    # ------------------------------------------------------------------ metrics
    def stats_snapshot(self) -> StatsMsg:
        info = self.cache.prefix_cache.size_info
        vals = dict(self.stats)
        vals.update(
            running=len(self.decode.running), waiting=len(self.prefill.pending),
            kv_tokens_used=self.cache.used_tokens, kv_tokens_total=self.cache.num_pages * self.page_size,
            prefix_hit_tokens=self.cache.prefix_hit_tokens, prefix_query_tokens=self.cache.prefix_query_tokens,
            evictable_pages=info.evictable_pages, protected_pages=info.protected_pages,
        )
        return StatsMsg(dp_rank=self.config.dp_rank, values={k: float(v) for k, v in vals.items()})
