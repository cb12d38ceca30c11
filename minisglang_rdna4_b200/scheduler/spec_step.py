"""One speculative decode step: propose → stage → verify → accept → commit
(python/minisgl/scheduler/scheduler.py:4755-5629).

Every running request feeds ``1 + K_i`` rows to one verify forward: its last committed token
followed by its draft. The target's arg-max (or distribution) of every row decides how many
draft tokens stand. Rejected rows leave stale KV behind; it is overwritten when those
positions are fed again, so only the length bookkeeping rolls back.
"""
from __future__ import annotations

import contextlib
from typing import List

import numpy as np
import torch

from ..core import Batch, Req
from ..engine import BatchSamplingArgs
from ..env import ENV
from ..message import DetokenizeMsg
from ..spec.accept import accept_greedy, accept_rejection_sampling, eos_truncate
from ..spec.width import AdaptiveWidth


def _engine_stream(eng):
    """Everything that touches the verify forward's results (logits, auxiliary hidden states,
    token pool, KV pool) is issued on the engine's stream: that stream does not synchronise
    with the default stream, so work left on the default stream could read the logits before
    the forward has produced them, and the next forward could read the token pool before the
    commit has landed."""
    if eng.device.type == "cuda":
        return torch.cuda.stream(eng.stream)
    return contextlib.nullcontext()


def req_spec_ok(sched, req: Req) -> bool:
    """May this request take a speculative step? The verify step accepts by arg-max (or, with
    ``MSGL_SPEC_SAMPLED``, by rejection sampling at a plain temperature); it applies no grammar
    mask, reasoning / tool-call gate, penalty, top-k / top-p / min-p filter or logprob
    capture. A request that needs any of those decodes one token at a time through the normal
    sampler (python/minisgl/scheduler/scheduler.py:3276-3293)."""
    sp = req.sampling_params
    if sched._needs_constraints(req) or sp.grammar is not None or sp.has_penalty or sp.logprobs > 0:
        return False
    if sp.is_greedy:
        return True
    if not ENV.SPEC_SAMPLED.value:
        return False
    return sp.top_k <= 0 and sp.top_p >= 1.0 and sp.min_p <= 0.0


def _verify_generator(sched, req: Req) -> torch.Generator:
    seed = req.sampling_params.seed if req.sampling_params.seed is not None else sched.config.seed * 1_000_003 + req.uid
    gen = torch.Generator(device="cpu")
    gen.manual_seed((int(seed) * 1_000_003 + req.num_generated) & 0x7FFFFFFFFFFFFFFF)
    return gen


def _plain_decode_step(sched) -> None:
    batch = sched.decode.schedule_next_batch()
    if batch is None:
        return
    ongoing = sched._forward(batch)
    sched._process_last_data(ongoing)
    proposer = sched.proposer
    if proposer is not None and hasattr(proposer, "on_plain_step"):
        proposer.on_plain_step(ongoing.sampled)


def spec_decode_step(sched) -> None:
    proposer = sched.proposer
    reqs: List[Req] = sorted(sched.decode.running.values(), key=lambda r: r.uid)
    if not reqs:
        return
    limit = ENV.SPEC_MAX_BS.value or proposer.max_batch
    if len(reqs) > limit or not all(req_spec_ok(sched, r) for r in reqs):
        _plain_decode_step(sched)
        return
    runner = device_runner(sched)
    with _engine_stream(sched.engine):
        if runner is not None and all(r.sampling_params.is_greedy for r in reqs):
            _device_spec_step(sched, proposer, runner, reqs)
        else:
            _spec_decode_step_on_stream(sched, proposer, reqs)


def device_runner(sched):
    """The GPU runner of the speculative step (``spec.device.DeviceSpecRunner``), built on first
    use: chain drafting with the n-gram proposer or the EAGLE3 / MTP head on a CUDA engine. Tree
    verification and CPU engines keep the host-driven step below."""
    runner = getattr(sched, "_spec_runner", False)
    if runner is not False:
        return runner
    runner = None
    eng, proposer = sched.engine, sched.proposer
    draft = getattr(proposer, "draft", None)
    tree_width = getattr(proposer, "tree_width", 1)
    # a tree on the device needs the draft head's ranked candidates; n-gram trees stay on the host-driven step
    # (models with recurrent layers roll their state back on the host-driven step)
    if (eng.device.type == "cuda" and not ENV.SPEC_HOST_STEP.value and (tree_width <= 1 or draft is not None)
            and proposer.num_draft >= 1 and eng.gdn_state is None and eng.swa is None
            and getattr(proposer, "device_step_ok", True)
            and not (sched.config.enable_ep and sched.config.dp_size > 1)):
        from ..spec.device import DeviceSpecRunner

        with _engine_stream(eng):
            runner = DeviceSpecRunner(eng, proposer.num_draft, draft, getattr(proposer, "capture_layers", None),
                                      max_batch=ENV.SPEC_MAX_BS.value or proposer.max_batch, tree_width=tree_width)
            runner.capture()
    sched._spec_runner = runner
    return runner


def _device_spec_step(sched, proposer, runner, reqs: List[Req]) -> None:
    """Host side of a step that runs entirely on the device: build the tables, replay, read the
    acceptance record, do the length bookkeeping and reply."""
    from ..utils import cdiv

    ps = sched.page_size
    K = runner.K
    host_drafts = runner.draft is None
    drafts = proposer.propose(reqs) if host_drafts else None
    rows, staged = [], []
    for i, r in enumerate(reqs):
        budget = proposer.budget(r)
        k = min(len(drafts[i]), budget) if host_drafts else budget
        c = r.cached_len
        end = r.device_len + k                      # positions c .. c + k get target K/V
        if runner.T > 1 and k > 0:
            # a tree also parks its siblings' K/V behind the chain; without room for them the request
            # takes a plain step (depth 0)
            if r.device_len + runner.K * runner.T <= sched.max_seq_len and k == runner.K:
                end = r.device_len + runner.K * runner.T
            else:
                k = 0
                end = r.device_len
        have = sched.alloc_len.get(r.uid, r.cache_handle.cached_len)
        if end > have:
            first, last = cdiv(have, ps), cdiv(end, ps)
            if last > first:
                sched.cache.page_table[r.table_idx, first:last] = sched.cache._take(last - first)
            sched.alloc_len[r.uid] = end
        n_pages = cdiv(end, ps)
        rows.append(dict(slot=r.table_idx, c=c, k=k, alloc_end=end, ignore_eos=r.sampling_params.ignore_eos,
                         max_emit=max(1, r.sampling_params.max_tokens - r.num_generated),
                         pages=sched.cache.page_table[r.table_idx, :n_pages]))
        staged.append(list(drafts[i][:k]) if host_drafts else [])
    record = runner.run(rows, staged)
    sched.stats["steps"] += 1
    sched.stats["spec_steps"] += 1
    sched.stats["decode_tokens"] += len(reqs) * runner.R
    replies: List[DetokenizeMsg] = []
    for i, r in enumerate(reqs):
        n, hit_eos = int(record[i, 0]), bool(record[i, 1])
        emitted = record[i, 2:2 + n].tolist()
        sched.stats["spec_drafted"] += rows[i]["k"]
        sched.stats["spec_accepted"] += n - 1
        sched.stats["spec_emitted"] += n
        r.append_host(torch.from_numpy(record[i, 2:2 + n].copy()))
        r.complete_many(n)
        proposer.on_accept(r, emitted)
        finished = hit_eos or r.num_generated >= r.sampling_params.max_tokens
        reason = "stop" if hit_eos else ("length" if finished else None)
        for j, t in enumerate(emitted):
            last = j == n - 1
            replies.append(DetokenizeMsg(r.uid, t, finished and last, reason if last else None,
                                         prompt_tokens=r.prompt_len, cached_tokens=sched.prefix_len.get(r.uid, 0)))
        if finished:
            r.finished, r.finish_reason = True, reason
            proposer.on_finish(r)
            sched._free_req_resources(r, insert=True)
    sched.decode.filter_finished()
    if replies:
        sched.send_result(replies)


def _spec_decode_step_on_stream(sched, proposer, reqs: List[Req]) -> None:
    if getattr(proposer, "tree_width", 1) > 1 and hasattr(proposer, "propose_paths") \
            and not getattr(proposer, "capture_layers", None):
        _tree_decode_step(sched, reqs)
        return
    for _ in _verify_phases(sched, proposer, reqs):
        pass


def spec_phases(sched, reqs: List[Req]):
    """The host-driven chain step in two halves, for loops that have to agree on a step's row count
    with other replicas before anybody launches (expert parallelism across replicas): the first
    ``next()`` proposes, stages the drafts and plans the verify forward, and yields its row count;
    exhausting the generator runs the forward and the acceptance."""
    proposer = sched.proposer
    with _engine_stream(sched.engine):
        gen = _verify_phases(sched, proposer, reqs)
        rows = next(gen)
    yield rows
    with _engine_stream(sched.engine):
        for _ in gen:
            pass


def _verify_phases(sched, proposer, reqs: List[Req]):
    if not hasattr(sched, "_spec_width"):
        sched._spec_width = AdaptiveWidth(proposer.num_draft)
    drafts = proposer.propose(reqs)
    width = sched._spec_width.choose() if ENV.SPEC_ADAPTIVE_WIDTH.value else proposer.num_draft
    drafts = [d[: min(width, proposer.budget(r))] for d, r in zip(drafts, reqs)]
    eng = sched.engine
    msl = sched.max_seq_len

    # stage the draft tokens behind each request's last token in the token pool
    flat_idx, flat_tok = [], []
    for r, d in zip(reqs, drafts):
        for j, t in enumerate(d):
            flat_idx.append(r.table_idx * msl + r.device_len + j)
            flat_tok.append(t)
    if flat_idx:
        idx = torch.tensor(flat_idx, dtype=torch.int64)
        tok = torch.tensor(flat_tok, dtype=torch.int32)
        eng.token_pool.view(-1)[idx.to(eng.device, non_blocking=True)] = tok.to(eng.device, non_blocking=True)

    batch = Batch(reqs=reqs, phase="decode")
    batch.spec_verify = True
    capture = getattr(proposer, "capture_layers", None)
    if capture:
        batch.capture_layers = list(capture)
    first_pos = [r.cached_len for r in reqs]
    plan = _verify_plan(sched, batch, drafts)
    sampled = any(not r.sampling_params.is_greedy for r in reqs) and ENV.SPEC_SAMPLED.value
    args = BatchSamplingArgs()
    rec = eng.gdn_state
    if rec is not None:
        # recurrent layers: the verify forward advances every request's state over all of its rows.
        # Keep the states as they are now and let every recurrent layer note its projected input, so
        # that the state of a request whose draft is cut short can be rebuilt over the kept rows
        rec_slots = torch.tensor([r.table_idx for r in reqs], dtype=torch.int64).to(eng.device)
        rec_saved = rec.save_slots(rec_slots)
        eng.ctx.recurrent_journal = []
    try:
        yield plan.num_tokens                     # planned; what follows launches and accepts
        out = eng.forward_batch(batch, plan, args, return_logits=True)
    finally:
        journal, eng.ctx.recurrent_journal = eng.ctx.recurrent_journal, None
    logits = eng.sampler.condition_logits(out.logits, args)
    aux = eng.ctx.aux_hidden if capture else None
    eng.ctx.aux_hidden = None
    target = logits.argmax(-1).to(torch.int32).cpu().tolist()
    sched.stats["steps"] += 1
    sched.stats["spec_steps"] += 1
    sched.stats["decode_tokens"] += plan.num_tokens

    replies: List[DetokenizeMsg] = []
    cu = plan.cu_q.tolist()
    total_accept = 0
    kept: List[int] = []
    for i, (r, d) in enumerate(zip(reqs, drafts)):
        rows = target[cu[i]:cu[i + 1]]
        if sampled and not r.sampling_params.is_greedy:
            temp = max(r.sampling_params.temperature, 1e-6)
            probs = torch.softmax(logits[cu[i]:cu[i + 1]].float() / temp, -1)
            # the uniforms come from a generator tied to (engine seed or request seed, request, tokens so
            # far): every tensor-parallel rank sees the same probabilities and so keeps the same tokens
            emitted = accept_rejection_sampling(probs, None, d, generator=_verify_generator(sched, r))
        else:
            emitted = accept_greedy(rows, d)
        emitted = emitted[: max(1, min(len(emitted), r.sampling_params.max_tokens - r.num_generated))]
        emitted, hit_eos = eos_truncate(emitted, sched.eos_ids, r.sampling_params.ignore_eos)
        n = len(emitted)
        kept.append(n)
        total_accept += n - 1
        sched.stats["spec_drafted"] += len(d)
        sched.stats["spec_accepted"] += n - 1
        sched.stats["spec_emitted"] += n
        # commit: tokens to the host buffer and (bonus token) to the token pool
        r.append_host(torch.tensor(emitted, dtype=torch.int32))
        pos = r.table_idx * msl + r.device_len
        eng.token_pool.view(-1)[pos:pos + n] = torch.tensor(emitted, dtype=torch.int32).to(eng.device)
        r.complete_many(n)
        if aux is not None and hasattr(proposer, "on_features"):
            rows = [a[cu[i]:cu[i] + n] for a in aux]
            proposer.on_features(r, rows, first_pos[i], torch.tensor(emitted, dtype=torch.int32))
        proposer.on_accept(r, emitted)
        finished = hit_eos or r.num_generated >= r.sampling_params.max_tokens
        reason = "stop" if hit_eos else ("length" if finished else None)
        for j, t in enumerate(emitted):
            last = j == n - 1
            replies.append(DetokenizeMsg(r.uid, t, finished and last, reason if last else None,
                                         prompt_tokens=r.prompt_len, cached_tokens=sched.prefix_len.get(r.uid, 0)))
        if finished:
            r.finished, r.finish_reason = True, reason
            proposer.on_finish(r)
            sched._free_req_resources(r, insert=True)
    if rec is not None:
        _rollback_recurrent(eng, journal, rec_slots, rec_saved, cu, kept, [r.finished for r in reqs])
    sched._spec_width.update(total_accept / max(len(reqs), 1))
    sched.decode.filter_finished()
    if replies:
        sched.send_result(replies)


def _rollback_recurrent(eng, journal, slots, saved, cu, kept, finished) -> None:
    """Recurrent state after a verify step (python/minisgl/gdn/layer.py:640-760 verify-replay): a
    request that kept all of its rows has the right state already. For the others the state from
    before the step is put back and every recurrent layer is advanced again over the kept rows
    only, from the projected inputs it noted during the verify forward; those inputs depend on
    earlier positions alone, so they are what a forward over just the kept rows would have seen."""
    part = [i for i, n in enumerate(kept) if n < cu[i + 1] - cu[i] and not finished[i]]
    if not part or not journal:
        return
    dev = eng.device
    which = torch.tensor(part, dtype=torch.int64).to(dev)
    eng.gdn_state.load_slots(slots, saved, which)
    rows = torch.tensor([cu[i] + j for i in part for j in range(kept[i])], dtype=torch.int64).to(dev)
    cu_new = torch.tensor(np.concatenate([[0], np.cumsum([kept[i] for i in part])]), dtype=torch.int32).to(dev)
    sub_slots = slots.index_select(0, which).to(torch.int32)
    has_state = torch.ones(len(part), dtype=torch.int32, device=dev)
    for layer, proj in journal:
        layer.replay(proj.index_select(0, rows), cu_new, sub_slots, has_state)


def _verify_plan(sched, batch: Batch, drafts):
    """Like ``Scheduler._make_plan`` but request i feeds ``1 + len(drafts[i])`` rows and every
    row is sampled."""
    from ..engine import StepPlan
    from ..utils import cdiv

    ps, msl = sched.page_size, sched.max_seq_len
    reqs = batch.reqs
    b = len(reqs)
    slots = np.fromiter((r.table_idx for r in reqs), dtype=np.int64, count=b)
    starts = np.fromiter((r.cached_len for r in reqs), dtype=np.int64, count=b)
    ends = np.fromiter((r.device_len + len(d) for r, d in zip(reqs, drafts)), dtype=np.int64, count=b)
    for r, end in zip(reqs, ends.tolist()):
        have = sched.alloc_len.get(r.uid, r.cache_handle.cached_len)
        if end > have:
            first, last = cdiv(have, ps), cdiv(end, ps)
            if last > first:
                sched.cache.page_table[r.table_idx, first:last] = sched.cache._take(last - first)
            sched.alloc_len[r.uid] = end
    swa = sched.engine.swa
    if swa is not None:
        # sliding-window pool: as in Scheduler._make_plan; pages of rejected draft rows simply stay with the
        # request and are written again when those positions are fed the next time
        for r, start, end in zip(reqs, starts.tolist(), ends.tolist()):
            swa.trim(r.table_idx, start)
            swa.ensure(r.table_idx, end)
    q_lens = ends - starts
    cu_q = np.zeros(b + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu_q[1:])
    total = int(cu_q[-1])
    row = np.repeat(slots, q_lens)
    pos = np.arange(total, dtype=np.int64) - np.repeat(cu_q[:-1].astype(np.int64), q_lens) + np.repeat(starts, q_lens)
    token_idx = (row * msl + pos).astype(np.int32)
    pages = sched.cache.page_table[row, pos // ps].astype(np.int64)
    out_loc = (pages * ps + pos % ps).astype(np.int32)
    max_kv = int(ends.max())
    block_table = np.ascontiguousarray(sched.cache.page_table[slots, : cdiv(max_kv, ps)], dtype=np.int32)
    return StepPlan(token_idx=token_idx, positions=pos.astype(np.int32), out_loc=out_loc, cu_q=cu_q,
                    seq_lens=ends.astype(np.int32), block_table=block_table,
                    sample_rows=np.arange(total, dtype=np.int32), write_idx=np.zeros(0, dtype=np.int32),
                    max_q=int(q_lens.max()), max_kv=max_kv)


def _tree_decode_step(sched, reqs: List[Req]) -> None:
    """Tree-structured verification (python/minisgl/spec/ddtree.py): the proposer's candidate
    continuations of a request are merged into a prefix tree; one forward scores every node, each
    attending to the committed prefix and to its ancestors through an additive mask; the target's
    arg-max is followed down the tree; the K/V of the accepted path are then moved to the
    positions they hold in the committed sequence. Greedy requests only (others take the
    target's token after the root, i.e. a plain decode step)."""
    from ..spec.tree import TokenTree, accept_greedy_tree, compaction_moves, tree_mask

    proposer = sched.proposer
    eng = sched.engine
    msl, ps = sched.max_seq_len, sched.page_size
    paths = proposer.propose_paths(reqs)
    max_nodes = 1 + proposer.num_draft * proposer.tree_width
    trees = []
    for r, cand in zip(reqs, paths):
        room = max(0, msl - r.device_len - 1)                 # KV slots left for draft nodes
        budget = min(proposer.budget(r), room)
        cand = [p[:budget] for p in cand] if r.sampling_params.is_greedy and budget > 0 else []
        trees.append(TokenTree.from_paths(0, cand, max_nodes=min(max_nodes, 1 + room)))

    # stage the node tokens behind each request's last token (node i at pool position cached_len + i)
    flat_idx, flat_tok = [], []
    for r, t in zip(reqs, trees):
        for i in range(1, len(t)):
            flat_idx.append(r.table_idx * msl + r.device_len - 1 + i)
            flat_tok.append(t.tokens[i])
    if flat_idx:
        idx = torch.tensor(flat_idx, dtype=torch.int64)
        tok = torch.tensor(flat_tok, dtype=torch.int32)
        eng.token_pool.view(-1)[idx.to(eng.device, non_blocking=True)] = tok.to(eng.device, non_blocking=True)

    batch = Batch(reqs=reqs, phase="decode")
    batch.spec_verify = True
    # rows and KV slots are laid out by node index; only the rotary positions follow the depth
    plan = _verify_plan(sched, batch, [[0] * (len(t) - 1) for t in trees])
    cu = plan.cu_q.tolist()
    prefix = [r.cached_len for r in reqs]
    pos = plan.positions.copy()
    mask = torch.full((plan.num_tokens, plan.max_kv), float("-inf"), dtype=torch.float32)
    for i, (t, p0) in enumerate(zip(trees, prefix)):
        pos[cu[i]:cu[i + 1]] = np.asarray([p0 + d for d in t.depth], dtype=pos.dtype)
        mask[cu[i]:cu[i + 1]] = tree_mask(t, p0, plan.max_kv)
    plan.positions[:] = pos
    batch.tree_mask = mask.to(eng.device)
    args = BatchSamplingArgs()
    out = eng.forward_batch(batch, plan, args, return_logits=True)
    logits = eng.sampler.condition_logits(out.logits, args)
    target = logits.argmax(-1).to(torch.int32).cpu().tolist()
    sched.stats["steps"] += 1
    sched.stats["spec_steps"] += 1
    sched.stats["decode_tokens"] += plan.num_tokens

    replies: List[DetokenizeMsg] = []
    buf = eng.kv_cache._buf
    for i, (r, t) in enumerate(zip(reqs, trees)):
        emitted, path = accept_greedy_tree(t, target[cu[i]:cu[i + 1]])
        emitted = emitted[: max(1, min(len(emitted), r.sampling_params.max_tokens - r.num_generated))]
        emitted, hit_eos = eos_truncate(emitted, sched.eos_ids, r.sampling_params.ignore_eos)
        n = len(emitted)
        sched.stats["spec_drafted"] += len(t) - 1
        sched.stats["spec_accepted"] += n - 1
        sched.stats["spec_emitted"] += n
        # accepted nodes' K/V -> the slots of their positions in the committed sequence
        row = sched.cache.page_table[r.table_idx]
        for src, dst in compaction_moves(path[:n], prefix[i]):
            buf[:, :, int(row[dst // ps]), :, dst % ps, :] = buf[:, :, int(row[src // ps]), :, src % ps, :]
        r.append_host(torch.tensor(emitted, dtype=torch.int32))
        at = r.table_idx * msl + r.device_len
        eng.token_pool.view(-1)[at:at + n] = torch.tensor(emitted, dtype=torch.int32).to(eng.device)
        r.complete_many(n)
        proposer.on_accept(r, emitted)
        finished = hit_eos or r.num_generated >= r.sampling_params.max_tokens
        reason = "stop" if hit_eos else ("length" if finished else None)
        for j, tok_id in enumerate(emitted):
            last = j == n - 1
            replies.append(DetokenizeMsg(r.uid, tok_id, finished and last, reason if last else None,
                                         prompt_tokens=r.prompt_len, cached_tokens=sched.prefix_len.get(r.uid, 0)))
        if finished:
            r.finished, r.finish_reason = True, reason
            proposer.on_finish(r)
            sched._free_req_resources(r, insert=True)
    sched.decode.filter_finished()
    if replies:
        sched.send_result(replies)
