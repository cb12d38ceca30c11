"""Speculative-decoding proposer interface (python/minisgl/spec/base.py:69,182)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import List, Sequence

import torch

from ..core import Req


class Proposer(ABC):
    """Proposes up to ``num_draft`` continuation tokens per running request."""

    name = "base"
    max_batch = 64   # above this batch size a plain decode step is cheaper than verifying

    def __init__(self, num_draft: int) -> None:
        self.num_draft = num_draft

    def budget(self, req: Req) -> int:
        """``K_i = min(num_draft, remain_len - 1)``: the verify step emits at most K+1 tokens
        (python/minisgl/spec/proposer.py:97)."""
        return max(0, min(self.num_draft, req.remain_len - 1))

    @abstractmethod
    def propose(self, reqs: Sequence[Req]) -> List[List[int]]:
        """One (possibly empty) draft token list per request."""

    def on_prefill(self, reqs: Sequence[Req]) -> None:
        """Called after a prefill step whose requests were sampled."""

    def on_accept(self, req: Req, emitted: Sequence[int]) -> None:
        """Called after tokens were committed to ``req``."""

    def on_finish(self, req: Req) -> None:
        """Called when ``req`` leaves the running set."""


def make_proposer(config, scheduler) -> Proposer:
    algo = config.spec_algorithm
    if algo == "ngram":
        from .ngram import NgramProposer

        return NgramProposer(config.spec_num_draft, config.spec_ngram_max, config.spec_ngram_min,
                             tree_width=max(1, int(getattr(config, "spec_tree_width", 1) or 1)))
    if algo in ("eagle3", "mtp"):
        from .gemma4_assistant import Gemma4AssistantProposer, is_gemma4_assistant

        if is_gemma4_assistant(getattr(config, "spec_draft_model_path", None)):
            # a drafter that reads the target's K/V (Gemma-4 "assistant" checkpoints)
            return Gemma4AssistantProposer(config, scheduler)
    if algo in ("eagle3", "mtp", "dflash"):
        from .dflash import DFlashProposer, is_dflash

        if algo == "dflash" or is_dflash(getattr(config, "spec_draft_model_path", None)):
            # a block-diffusion drafter: one forward proposes the whole chain
            return DFlashProposer(config, scheduler)
    if algo == "tidar":
        from .tidar import TiDARProposer

        return TiDARProposer(config, scheduler)
    if algo == "eagle3":
        from .eagle3 import Eagle3Proposer

        return Eagle3Proposer(config, scheduler)
    if algo == "mtp":
        mc = scheduler.engine.model_config
        qwen = mc.mtp_num_hidden_layers > 0 and mc.attn_output_gate and mc.layer_types
        glm = mc.num_nextn_predict_layers > 0 and (getattr(mc, "kv_lora_rank", 0) or mc.model_type == "glm4_moe")
        if qwen or glm:
            # the checkpoint's own head (Qwen3.5 / Qwen3-Next mtp.*; GLM-4.x MoE / DeepSeek model.layers.<L>)
            from .mtp import MTPProposer

            return MTPProposer(config, scheduler)
        from .eagle3 import Eagle3Proposer

        return Eagle3Proposer(config, scheduler, mtp=True)
    raise ValueError(f"unknown speculative algorithm {algo!r}")
