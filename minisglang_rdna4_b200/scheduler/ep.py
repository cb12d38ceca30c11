"""Lock-step scheduling loop for expert parallelism across replicas
(python/minisgl/scheduler/ep.py:17-172).

The MoE layers of every replica exchange rows each forward, so all replicas must run a
forward at the same time and with the same padded row count. Each iteration the replicas
all-reduce (MAX, over the gloo group of their column) ``[tokens of my step, exit flag]``;
a replica with nothing to do runs a one-token dummy step that writes only the dummy KV page.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ..core import Batch
from ..engine import BatchSamplingArgs, StepPlan
from ..env import ENV


def _dummy_step(sched) -> None:
    """Forward one token of the dummy request: keeps this replica inside the collectives."""
    eng = sched.engine
    slot = eng.num_slots - 1
    dummy_loc = eng.kv_cache.dummy_page * eng.page_size
    plan = StepPlan(
        token_idx=np.array([slot * eng.max_seq_len], dtype=np.int32), positions=np.zeros(1, dtype=np.int32),
        out_loc=np.array([dummy_loc], dtype=np.int32), cu_q=np.array([0, 1], dtype=np.int32),
        seq_lens=np.ones(1, dtype=np.int32),
        block_table=np.full((1, 1), eng.kv_cache.dummy_page, dtype=np.int32),
        sample_rows=np.zeros(0, dtype=np.int32), write_idx=np.zeros(0, dtype=np.int32), max_q=1, max_kv=1)
    batch = Batch(reqs=[], phase="prefill")
    eng.forward_batch(batch, plan, BatchSamplingArgs())


def ep_lockstep_loop(sched) -> None:
    from .scheduler import RequestAllFinished

    eng = sched.engine
    group = eng.dp_cpu_group
    ep = eng.ctx.ep
    idle_rounds = 0
    local_done = False
    steps = 0
    health_every = max(1, ENV.COMM_HEALTH_STEPS.value)
    while True:
        # a replica whose own requests are all finished keeps stepping with the others (their tokens
        # may be routed to its experts) until every replica agrees that nothing is left
        try:
            for msg in ([] if local_done else sched.receive_msg(blocking=False)):
                sched._process_one_msg(msg)
        except RequestAllFinished:
            local_done = True
        # a replica whose running requests can all take a speculative step proposes and plans it first, so
        # that its row count (1 + draft length per request) goes into the agreement
        spec = None
        batch = None
        tokens = 0
        if sched.proposer is not None and not sched.prefill.runnable and sched.decode.runnable:
            from .spec_step import req_spec_ok, spec_phases

            reqs = sorted(sched.decode.running.values(), key=lambda r: r.uid)
            limit = ENV.SPEC_MAX_BS.value or sched.proposer.max_batch
            if reqs and len(reqs) <= limit and all(req_spec_ok(sched, r) for r in reqs) and getattr(
                    sched.proposer, "tree_width", 1) <= 1:
                spec = spec_phases(sched, reqs)
                tokens = next(spec)
        if spec is None:
            batch = sched._schedule_next_batch()
            if batch is not None:
                tokens = sum(r.extend_len for r in batch.reqs)
        # the status word of the peer-memory exchange rides along every few steps (the host has
        # synchronised with the device at the end of the previous step, so the read does not stall)
        poll = getattr(ep, "poll_status", None)
        status = poll() if poll is not None and steps % health_every == 0 else 0
        agree = torch.tensor([tokens, 1 if sched._exit else 0,
                              1 if ((sched.has_work or batch is not None or spec is not None)
                                    and not (local_done and batch is None and spec is None)) else 0,
                              status], dtype=torch.int64)
        dist.all_reduce(agree, op=dist.ReduceOp.MAX, group=group)
        common, any_exit, any_work = int(agree[0]), int(agree[1]), int(agree[2])
        if int(agree[3]) != 0 and getattr(ep, "healthy", False):
            # a bounded wait ran out on some replica (a peer was more than the limit late): rows of
            # the steps since the last clean check may be missing from somebody's sums. Every
            # replica leaves the fused exchange on this step, decode leaves its captured graphs
            # (they contain the exchange kernels) and the running requests end with an error.
            ep.healthy = False
            eng.graph_runner = None
            sched._fail_running("the expert exchange timed out; the request was ended because its state may be incomplete")
            batch = None if batch is not None and all(r.finished for r in batch.reqs) else batch
            if spec is not None:
                spec.close()                       # its requests were just ended: run a dummy step instead
                spec = None
        if common == 0:
            if any_exit and not any_work:
                break
            # nobody has a step to run: in offline mode that means everything is finished
            if getattr(sched.config, "offline_mode", False) and not any_work:
                break
            idle_rounds += 1
            if idle_rounds > 2:
                import time

                time.sleep(0.002)
            continue
        idle_rounds = 0
        ep.common_tokens = common
        if spec is not None:
            for _ in spec:                         # verify forward (rows exchanged with the other replicas) + acceptance
                pass
        elif batch is not None:
            ongoing = sched._forward(batch)
            sched._process_last_data(ongoing)
            if sched.proposer is not None and batch.is_prefill:
                sched._feed_prefill_features(batch)
                sched.proposer.on_prefill(ongoing.sampled)
        else:
            _dummy_step(sched)
        ep.common_tokens = None
        steps += 1
        sched._maybe_exit_after_steps()
