"""TiDAR: the target drafts for itself (python/minisgl/spec/tidar.py:1-120,
python/minisgl/scheduler/scheduler.py:3630-3790).

A TiDAR-trained model answers mask tokens behind its text with the tokens that belong there. One causal
forward of the TARGET over ``[confirmed token, mask x k]`` per request gives ``k`` drafts (the arg-max at the
mask rows); the ordinary chain verification then runs over ``[confirmed token, drafts]``. The drafting
forward leaves nothing behind: its rows go to the K/V slots the verification rows are about to overwrite,
request lengths do not move, nothing is sampled or written back to the token pool's committed part.

No draft checkpoint and no draft state. ``tidar_config.json`` (draft path or model directory) names the
mask token and the trained block size. Models with recurrent layers are refused (the drafting forward would
advance their state), and so is the sliding-window pool (its page recycling follows committed lengths).
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Sequence

import torch

from ..core import Batch, Req
from .base import Proposer


def tidar_config(*paths) -> dict:
    for p in paths:
        if p and os.path.isfile(os.path.join(p, "tidar_config.json")):
            with open(os.path.join(p, "tidar_config.json")) as fh:
                return json.load(fh)
    return {}


class TiDARProposer(Proposer):
    name = "tidar"
    device_step_ok = False

    def __init__(self, config, scheduler) -> None:
        super().__init__(config.spec_num_draft)
        # > 1: a draft tree from the top tokens of every position instead of the arg-max chain
        self.tree_width = max(1, int(getattr(config, "spec_tree_width", 1) or 1))
        self.sched, self.engine = scheduler, scheduler.engine
        raw = tidar_config(getattr(config, "spec_draft_model_path", None), config.model_path)
        mask = raw.get("mask_token_id", self.engine.model_config.mask_token_id)
        if mask is None:
            raise ValueError("TiDAR needs a mask token: tidar_config.json (mask_token_id) or the model config")
        self.mask_token_id = int(mask)
        self.block = int(raw.get("block_size") or 0) or self.num_draft
        if self.engine.gdn_state is not None or self.engine.swa is not None:
            raise NotImplementedError("TiDAR self-drafting needs a target without recurrent layers and without the "
                                      "sliding-window pool")

    def propose(self, reqs: Sequence[Req]) -> List[List[int]]:
        return [lp.argmax(-1).tolist() if lp is not None else [] for lp in self._block_logits(reqs)]

    def propose_paths(self, reqs: Sequence[Req]) -> List[List[List[int]]]:
        """Per request the most probable prefixes under the per-position distributions of the drafting
        forward (``spec/ddtree.py``), best first: ``num_draft x tree_width`` tree nodes from the top
        ``tree_width`` tokens of every position."""
        from .ddtree import build_draft_paths

        out = []
        for lp in self._block_logits(reqs):
            if lp is None:
                out.append([])
                continue
            val, idx = torch.log_softmax(lp, -1).topk(min(self.tree_width, lp.shape[-1]), -1)
            out.append(build_draft_paths(val.tolist(), idx.tolist(), self.num_draft * self.tree_width))
        return out

    def _block_logits(self, reqs: Sequence[Req]) -> List[Optional[torch.Tensor]]:
        """One drafting forward; per request the fp32 logits ``[k_i, vocab]`` of its mask rows (``None`` for a
        request with no budget)."""
        from ..engine import BatchSamplingArgs
        from ..scheduler.spec_step import _engine_stream

        out: List[Optional[torch.Tensor]] = [None for _ in reqs]
        rows = [i for i, r in enumerate(reqs) if min(self.budget(r), self.block) > 0]
        if not rows:
            return out
        eng, sched = self.engine, self.sched
        mine = [reqs[i] for i in rows]
        k = max(min(self.budget(r), self.block) for r in mine)
        k = min(k, min(sched.max_seq_len - r.device_len for r in mine))
        if k <= 0:
            return out
        msl = sched.max_seq_len
        # the masks go behind the confirmed token in the token pool (positions the verification rewrites)
        idx = torch.cat([torch.arange(r.table_idx * msl + r.device_len, r.table_idx * msl + r.device_len + k)
                         for r in mine])
        batch = Batch(reqs=mine, phase="decode")
        batch.spec_verify = True                  # every row yields logits, nothing is written back
        plan = sched._make_plan(batch, extra_rows=k)
        with _engine_stream(eng):
            eng.token_pool.view(-1)[idx.to(eng.device)] = self.mask_token_id
            res = eng.forward_batch(batch, plan, BatchSamplingArgs(), return_logits=True)
            logits = eng.sampler.condition_logits(res.logits, BatchSamplingArgs())
            logits = logits.float().cpu()
        cu = plan.cu_q.tolist()
        for j, i in enumerate(rows):
            first = cu[j + 1] - k                  # the mask rows are the last k of the request
            out[i] = logits[first:first + min(self.budget(reqs[i]), self.block, k)]
        sched.stats["steps"] += 1
        return out
