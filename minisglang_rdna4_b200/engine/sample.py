"""Sampler: turns last-token logits into token ids.

Order of operations (python/minisgl/engine/sample.py:108-142,146-437): NaN fence →
final-logit soft cap → padded-vocabulary fence → log-prob capture → grammar bitmask →
presence/frequency penalties over the tokens a request has generated → greedy arg-max or
temperature / min-p / top-k / top-p sampling. Under tensor parallelism every rank computes
the same logits; the ids of rank 0 are adopted by all ranks so that a non-deterministic
reduction order can never make ranks diverge.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..core import Req
from ..env import ENV


@dataclass
class BatchSamplingArgs:
    temperatures: Optional[torch.Tensor] = None   # None = whole batch greedy
    top_k: Optional[torch.Tensor] = None
    top_p: Optional[torch.Tensor] = None
    min_p: Optional[torch.Tensor] = None
    penalty_rows: Optional[torch.Tensor] = None   # rows that carry a penalty
    penalty_tokens: Optional[torch.Tensor] = None  # [n_pen, max_gen] generated ids padded with -1
    presence: Optional[torch.Tensor] = None
    frequency: Optional[torch.Tensor] = None
    logprobs: int = 0
    bitmask: Optional[torch.Tensor] = None        # [bs, ceil(V/32)] int32 allowed-token bits
    bitmask_rows: Optional[torch.Tensor] = None
    generators: Optional[List[Optional[torch.Generator]]] = None
    seeded_uniform: Optional[torch.Tensor] = None  # [bs] draw of every request that carries a seed, NaN elsewhere

    @property
    def greedy(self) -> bool:
        return self.temperatures is None


@dataclass
class SampleOutput:
    tokens: torch.Tensor
    logprobs: Optional[torch.Tensor] = None        # [bs] log-prob of the chosen token
    top_logprobs: Optional[torch.Tensor] = None    # [bs, n]
    top_ids: Optional[torch.Tensor] = None


class Sampler:
    def __init__(self, device, vocab_size: int, softcap: Optional[float] = None, seed: int = 0) -> None:
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.softcap = softcap
        self.generator = torch.Generator(device=self.device)
        self.generator.manual_seed(seed)
        self.nan_events = 0

    # ---- host side: build the per-batch tensors ----
    def prepare(self, reqs: Sequence[Req]) -> BatchSamplingArgs:
        params = [r.sampling_params for r in reqs]
        args = BatchSamplingArgs()
        args.logprobs = max((p.logprobs for p in params), default=0)
        if not all(p.is_greedy for p in params):
            dev = self.device
            args.temperatures = torch.tensor(
                [0.0 if p.is_greedy else p.temperature for p in params], dtype=torch.float32).to(dev, non_blocking=True)
            if any(p.top_k > 0 for p in params):
                args.top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(dev, non_blocking=True)
            if any(p.top_p < 1.0 for p in params):
                args.top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32).to(dev, non_blocking=True)
            if any(p.min_p > 0.0 for p in params):
                args.min_p = torch.tensor([p.min_p for p in params], dtype=torch.float32).to(dev, non_blocking=True)
            if any(p.seed is not None for p in params):
                # a request with a seed draws u = f(seed, index of the token): the same request gives the
                # same text whatever it is batched with (python/minisgl/engine/sample.py, per-request seed)
                import numpy as np

                u = [float("nan") if p.seed is None else
                     float(np.random.default_rng([int(p.seed) & 0x7FFFFFFF, r.num_generated]).random())
                     for p, r in zip(params, reqs)]
                args.seeded_uniform = torch.tensor(u, dtype=torch.float32).to(dev, non_blocking=True)
        pen = [i for i, p in enumerate(params) if p.has_penalty and reqs[i].num_generated > 0]
        if pen:
            width = max(reqs[i].num_generated for i in pen)
            toks = torch.full((len(pen), width), -1, dtype=torch.int64)
            for row, i in enumerate(pen):
                g = reqs[i].generated_ids
                toks[row, : g.numel()] = g
            dev = self.device
            args.penalty_rows = torch.tensor(pen, dtype=torch.int64).to(dev)
            args.penalty_tokens = toks.to(dev)
            args.presence = torch.tensor([params[i].presence_penalty for i in pen], dtype=torch.float32).to(dev)
            args.frequency = torch.tensor([params[i].frequency_penalty for i in pen], dtype=torch.float32).to(dev)
        return args

    # ---- device side ----
    def condition_logits(self, logits: torch.Tensor, args: BatchSamplingArgs) -> torch.Tensor:
        """Everything that edits logits before the draw; also used on speculative verify rows."""
        if ENV.SANITIZE_LOGITS.value:
            bad = ~torch.isfinite(logits)
            if bool(bad.any()):
                self.nan_events += 1
                logits = torch.where(bad, torch.full_like(logits, -1e30), logits)
        if self.softcap:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        if logits.shape[-1] > self.vocab_size:
            logits = logits[:, : self.vocab_size]
        if args.bitmask is not None:
            logits = apply_token_bitmask(logits, args.bitmask, args.bitmask_rows)
        if args.penalty_rows is not None:
            logits = apply_penalties(logits, args.penalty_rows, args.penalty_tokens, args.presence, args.frequency)
        return logits

    def sample(self, logits: torch.Tensor, args: BatchSamplingArgs) -> SampleOutput:
        out = SampleOutput(tokens=None)  # type: ignore[arg-type]
        if args.logprobs > 0:
            # the model's own distribution: after soft cap and vocabulary fence, before masks/penalties
            raw = logits[:, : self.vocab_size].float()
            if self.softcap:
                raw = torch.tanh(raw / self.softcap) * self.softcap
            lp = torch.log_softmax(raw, dim=-1)
            out.top_logprobs, out.top_ids = lp.topk(args.logprobs, dim=-1)
        logits = self.condition_logits(logits, args)
        if args.greedy:
            out.tokens = ops.argmax(logits)
        else:
            uniform = None
            if args.seeded_uniform is not None:
                uniform = torch.rand((logits.shape[0],), dtype=torch.float32, device=logits.device,
                                     generator=self.generator)
                uniform = torch.where(torch.isnan(args.seeded_uniform), uniform, args.seeded_uniform)
            out.tokens = ops.sample(logits, args.temperatures, args.top_k, args.top_p, args.min_p,
                                    generator=self.generator, uniform=uniform)
        if args.logprobs > 0:
            out.logprobs = lp.gather(-1, out.tokens.long()[:, None]).squeeze(-1)
        return out


def apply_penalties(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor,
                    presence: torch.Tensor, frequency: torch.Tensor) -> torch.Tensor:
    """``logit -= presence * [count > 0] + frequency * count`` over generated tokens
    (python/minisgl/engine/sample.py:224-250)."""
    vocab = logits.shape[-1]
    valid = tokens >= 0
    counts = torch.zeros((tokens.shape[0], vocab), dtype=torch.float32, device=logits.device)
    counts.scatter_add_(1, tokens.clamp_min(0), valid.float())
    delta = presence[:, None] * (counts > 0).float() + frequency[:, None] * counts
    logits = logits.clone() if logits.dtype == torch.float32 else logits.float()
    logits[rows] = logits[rows] - delta
    return logits


def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor, rows: Optional[torch.Tensor]) -> torch.Tensor:
    """Set logits of tokens whose bit is 0 to -inf. ``bitmask`` ``[n, ceil(V/32)]`` int32."""
    vocab = logits.shape[-1]
    bits = torch.arange(32, device=logits.device, dtype=torch.int32)
    allowed = ((bitmask[:, :, None] >> bits) & 1).bool().reshape(bitmask.shape[0], -1)[:, :vocab]
    logits = logits.clone()
    if rows is None:
        logits.masked_fill_(~allowed, float("-inf"))
    else:
        sub = logits[rows]
        sub.masked_fill_(~allowed, float("-inf"))
        logits[rows] = sub
    return logits
