"""Denoising schedule and canvas state of block-diffusion decoding
(python/minisgl/diffusion/sampler.py:1-594).

A block-diffusion model writes ``block`` tokens at once: the block's positions (the canvas) are fed
together, attend to each other in both directions and to the committed context causally, and the
canvas is refined over a few forwards. Two refinement rules are built:

``entropy_bound`` (uniform-state diffusion, the reference's DiffusionGemma rule). The canvas starts
as uniform-random token ids; there is no mask token. Every step, with ``T`` falling linearly from
``t_max`` to ``t_min`` as the step counter counts down:

* ``p = softmax(logits / T)`` (computed as the softmax of the log-normalised logits, the way
  ``torch.distributions.Categorical`` does, because the entropies are sorted and a last-bit
  difference can flip the order), ``H`` its entropy per position;
* the positions are ordered by entropy and the longest prefix whose entropies, without its largest,
  sum to at most ``entropy_bound`` takes a token drawn from ``p``; every other position is
  re-drawn uniformly (a position accepted in one step may be noise again in the next: the
  incoming canvas is not read at all);
* the candidate output is the arg-max canvas, not the sampled one; the block ends early once the
  arg-max canvas has been the same for ``stability_threshold`` steps and the mean entropy is below
  ``confidence_threshold``, or when the steps run out. The arg-max canvas is what is committed.

``mask_confidence`` (absorbing-state diffusion, the LLaDA / SDAR family). The canvas starts as the
mask token everywhere; every step each masked position proposes its most likely token (or a draw at
a temperature), and the positions whose proposal has probability of at least ``unmask_threshold``
are filled in, at least the most confident one and at least as many as are needed to finish within
the remaining steps. Filled positions stay. The block ends when no mask is left.

All draws of a request come from one generator seeded from the request's seed (or the engine seed
and the request id), so tensor-parallel ranks, which see identical logits, make identical draws.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass(frozen=True)
class DenoiseConfig:
    kind: str                         # "entropy_bound" | "mask_confidence"
    block: int                        # canvas length
    vocab_size: int
    max_steps: int
    t_min: float = 0.0
    t_max: float = 0.0
    entropy_bound: float = 0.0
    confidence_threshold: float = 0.0
    stability_threshold: int = 0
    mask_token_id: Optional[int] = None
    unmask_threshold: float = 0.9

    def temperature(self, steps_left: int) -> float:
        """``steps_left`` counts down from ``max_steps`` to 1: the first step is the hottest."""
        return self.t_min + (self.t_max - self.t_min) * (steps_left / self.max_steps)

    @classmethod
    def from_model(cls, model_path: Optional[str], model_config, overrides: Optional[dict] = None) -> "DenoiseConfig":
        """From the checkpoint's ``generation_config.json`` (the schedule is a property of the model:
        a wrong bound or threshold still yields fluent text, so missing keys are an error, not a
        default) and ``config.json`` (``canvas_length``, ``mask_token_id``)."""
        gen = {}
        if model_path and os.path.isfile(os.path.join(model_path, "generation_config.json")):
            with open(os.path.join(model_path, "generation_config.json")) as f:
                gen = json.load(f)
        gen.update(overrides or {})
        block = int(gen.get("canvas_length") or model_config.canvas_length or 0)
        if block <= 0:
            raise ValueError("block-diffusion decoding needs canvas_length (config.json)")
        sampler = gen.get("sampler_config") or {}
        name = sampler.get("_cls_name", "")
        mask_id = gen.get("mask_token_id", model_config.mask_token_id)
        if name == "EntropyBoundSamplerConfig" or (not name and mask_id is None):
            need = ("max_denoising_steps", "t_min", "t_max", "confidence_threshold", "stability_threshold")
            missing = [k for k in need if k not in gen] + ([] if "entropy_bound" in sampler else ["sampler_config.entropy_bound"])
            if missing:
                raise ValueError(f"the denoising schedule is incomplete: generation_config.json lacks {missing}")
            return cls("entropy_bound", block, int(model_config.vocab_size), int(gen["max_denoising_steps"]),
                       float(gen["t_min"]), float(gen["t_max"]), float(sampler["entropy_bound"]),
                       float(gen["confidence_threshold"]), int(gen["stability_threshold"]))
        if mask_id is None:
            raise ValueError(f"diffusion sampler {name!r} needs mask_token_id")
        return cls("mask_confidence", block, int(model_config.vocab_size),
                   int(gen.get("max_denoising_steps") or gen.get("denoising_steps") or block),
                   float(gen.get("t_min", 0.0)), float(gen.get("t_max", 0.0)), mask_token_id=int(mask_id),
                   unmask_threshold=float(gen.get("confidence_threshold", sampler.get("threshold", 0.9))))


def entropy_bound_accept(entropy: torch.Tensor, bound: float) -> torch.Tensor:
    """Positions of the longest ascending-entropy prefix whose entropies minus the largest of them
    sum to at most ``bound``. The lowest-entropy position always qualifies."""
    order = torch.argsort(entropy)
    ranked = entropy[order]
    ok = torch.cumsum(ranked, 0) - ranked <= bound
    out = torch.zeros_like(ok)
    out[order] = ok
    return out


class Canvas:
    """One request's block in progress. ``tokens`` is what the next forward is fed, ``emit`` what
    would be committed if the block ended now."""

    def __init__(self, cfg: DenoiseConfig, length: int, device, generator: Optional[torch.Generator] = None) -> None:
        self.cfg, self.length, self.device = cfg, int(length), torch.device(device)
        self.generator = generator
        self.steps_left = cfg.max_steps
        self.steps_taken = 0
        self.finished = False
        self.mean_entropy = float("nan")
        # models with self-conditioning: the distribution every row predicted in the last step is kept for
        # the caller (which turns it into the next step's signal and clears it)
        self.keep_probs = False
        self.probs: Optional[torch.Tensor] = None
        self.signal: Optional[torch.Tensor] = None
        self._history: List[torch.Tensor] = []
        if cfg.kind == "entropy_bound":
            self.tokens = self._noise()
        else:
            self.tokens = torch.full((self.length,), int(cfg.mask_token_id), dtype=torch.int64, device=self.device)
        self.emit = self.tokens.clone()

    def _noise(self) -> torch.Tensor:
        return torch.randint(0, self.cfg.vocab_size, (self.length,), device=self.device, generator=self.generator)

    def advance(self, logits: torch.Tensor) -> None:
        """``logits`` ``[length, vocab]`` of this request's canvas rows (fp32, soft cap applied)."""
        assert not self.finished, "a finished block is not stepped again"
        logits = logits.float()
        if self.cfg.kind == "entropy_bound":
            self._advance_entropy_bound(logits)
        else:
            self._advance_mask_confidence(logits)
        self.steps_left -= 1
        self.steps_taken += 1
        if self.steps_left <= 0:
            self.finished = True

    # ---- uniform-state rule ----
    def _advance_entropy_bound(self, logits: torch.Tensor) -> None:
        cfg = self.cfg
        scaled = logits / cfg.temperature(self.steps_left)
        logp = scaled - scaled.logsumexp(-1, keepdim=True)
        p = torch.softmax(logp, -1)
        entropy = -(p * logp).sum(-1)
        if self.keep_probs:
            self.probs = p
        top = scaled.argmax(-1)
        drawn = torch.multinomial(p, 1, generator=self.generator).squeeze(-1)     # before the re-noise: draw order
        fresh = self._noise()
        accepted = entropy_bound_accept(entropy, cfg.entropy_bound)
        self.tokens = torch.where(accepted, drawn, fresh)
        self.emit = top
        k = cfg.stability_threshold
        stable = k == 0 or (len(self._history) >= k and all(torch.equal(h, top) for h in self._history))
        self._history.append(top)
        if len(self._history) > k:
            self._history.pop(0)
        self.mean_entropy = float(entropy.mean())
        if stable and self.mean_entropy < cfg.confidence_threshold:
            self.finished = True

    # ---- absorbing-state rule ----
    def _advance_mask_confidence(self, logits: torch.Tensor) -> None:
        cfg = self.cfg
        masked = self.tokens == int(cfg.mask_token_id)
        n_masked = int(masked.sum())
        if n_masked == 0:
            self.finished = True
            return
        t = cfg.temperature(self.steps_left)
        p = torch.softmax(logits, -1)
        if self.keep_probs:
            self.probs = p
        if t > 0:
            choice = torch.multinomial(torch.softmax(logits / t, -1), 1, generator=self.generator).squeeze(-1)
        else:
            choice = logits.argmax(-1)
        choice = torch.where(choice == int(cfg.mask_token_id), logits.topk(2, -1).indices[:, 1], choice)
        conf = p.gather(-1, choice[:, None]).squeeze(-1)
        conf = torch.where(masked, conf, torch.full_like(conf, -1.0))
        need = max(1, math.ceil(n_masked / max(self.steps_left, 1)))             # finish within the steps
        count = max(need, int((conf >= cfg.unmask_threshold).sum()))
        pick = torch.topk(conf, min(count, n_masked)).indices
        self.tokens = self.tokens.clone()
        self.tokens[pick] = choice[pick]
        self.emit = torch.where(self.tokens == int(cfg.mask_token_id), choice, self.tokens)
        self.mean_entropy = float(-(p * torch.log(p.clamp_min(1e-30))).sum(-1).mean())
        if not bool((self.tokens == int(cfg.mask_token_id)).any()):
            self.finished = True
