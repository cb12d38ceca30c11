"""Offline generation API: ``LLM(...).generate(prompts, sampling_params)``.

The scheduler runs in-process with its message hooks replaced by a local queue
(python/minisgl/llm/llm.py:30-147). Prompts are lists of token ids, or strings when a
tokenizer is available for the model path.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from .config import SchedulerConfig
from .core import SamplingParams
from .message import BaseMsg, DetokenizeMsg, UserMsg
from .scheduler import RequestAllFinished, Scheduler


@dataclass
class RequestOutput:
    uid: int
    prompt_token_ids: List[int]
    token_ids: List[int] = field(default_factory=list)
    text: Optional[str] = None
    finish_reason: Optional[str] = None
    logprobs: List[float] = field(default_factory=list)
    cached_tokens: int = 0
    error: Optional[str] = None


class LLM(Scheduler):
    def __init__(self, model_path: str = "", **kwargs: Any) -> None:
        from .utils.hub import resolve_model_path

        model_path = resolve_model_path(model_path) or ""
        if kwargs.get("spec_draft_model_path"):
            kwargs["spec_draft_model_path"] = resolve_model_path(kwargs["spec_draft_model_path"])
        config = kwargs.pop("config", None)
        if config is None:
            config = SchedulerConfig(model_path=model_path, offline_mode=True, **kwargs)
        else:
            config = dataclasses.replace(config, offline_mode=True)
        super().__init__(config)
        self._queue: List[UserMsg] = []
        self._outputs: Dict[int, RequestOutput] = {}
        self._unfinished = 0
        self._next_uid = 0
        self._tokenizer = None

    # ---- scheduler hooks ----
    def receive_msg(self, blocking: bool) -> List[BaseMsg]:
        if not self._queue:
            if self._unfinished == 0:
                raise RequestAllFinished()
            return []
        # feed at most one prefill budget of prompt tokens per poll
        budget = self.config.max_extend_tokens
        out: List[BaseMsg] = []
        while self._queue and (budget > 0 or not out):
            msg = self._queue.pop(0)
            budget -= int(msg.input_ids.numel())
            out.append(msg)
        return out

    def send_result(self, replies: List[DetokenizeMsg]) -> None:
        for r in replies:
            out = self._outputs[r.uid]
            if r.error is not None:
                out.error = r.error
            else:
                out.token_ids.append(r.next_token)
                if r.logprob is not None:
                    out.logprobs.append(r.logprob)
            out.cached_tokens = r.cached_tokens
            if r.finished:
                out.finish_reason = r.finish_reason
                self._unfinished -= 1

    # ---- public ----
    def _get_tokenizer(self):
        if self._tokenizer is None:
            from transformers import AutoTokenizer

            self._tokenizer = AutoTokenizer.from_pretrained(self.config.model_path)
        return self._tokenizer

    def generate(self, prompts: Sequence[Union[str, Sequence[int], torch.Tensor]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 images: Optional[Sequence] = None) -> List[RequestOutput]:
        """``images``: per prompt ``None`` or a list of images (encoded bytes, PIL images or uint8
        tensors). A token-id prompt carries one begin-of-image marker per image; the placeholder
        tokens are filled in here."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        uids = []
        for prompt, sp in zip(prompts, sampling_params):
            if isinstance(prompt, str):
                ids = torch.tensor(self._get_tokenizer().encode(prompt), dtype=torch.int32)
            else:
                ids = torch.as_tensor(prompt, dtype=torch.int32).reshape(-1)
            uid = self._next_uid
            self._next_uid += 1
            uids.append(uid)
            pixels = None
            mine = images[len(uids) - 1] if images is not None else None
            if mine:
                from .tokenizer.vision import VisionPreprocessor

                vc = self.engine.model_config.vision
                if vc is None:
                    raise ValueError("this model takes no image input")
                pre = VisionPreprocessor.from_vision_config(vc)
                pixels = pre.batch(mine)
                ids = torch.tensor(pre.expand_placeholders(ids.tolist(), len(mine)), dtype=torch.int32)
            self._outputs[uid] = RequestOutput(uid, ids.tolist())
            self._queue.append(UserMsg(uid, ids, sp, images=pixels))
            self._unfinished += 1
        self._exit = False
        self.run_forever()
        outs = [self._outputs.pop(u) for u in uids]
        if self._tokenizer is not None:
            for o in outs:
                o.text = self._tokenizer.decode(o.token_ids, skip_special_tokens=True)
        return outs

    def shutdown(self) -> None:
        self.engine.shutdown()
