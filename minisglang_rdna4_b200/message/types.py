"""Message dataclasses (python/minisgl/message/backend.py:12-59, frontend.py:9-81,
tokenizer.py:11-121). Every message is a flat dataclass so the msgpack codec can rebuild it
from its class name and field dict."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ..core import SamplingParams


@dataclass
class BaseMsg:
    pass


# ---- frontend → tokenizer ----
@dataclass
class TokenizeMsg(BaseMsg):
    uid: int
    text: Any                       # str prompt or list of chat messages
    sampling_params: SamplingParams
    chat_template_kwargs: Optional[Dict[str, Any]] = None
    tools: Optional[List[Dict[str, Any]]] = None
    add_generation_prompt: bool = True
    images: Optional[List[bytes]] = None    # encoded image files, in the order their placeholders appear


@dataclass
class AbortMsg(BaseMsg):
    uid: int


# ---- tokenizer → scheduler ----
@dataclass
class UserMsg(BaseMsg):
    uid: int
    input_ids: torch.Tensor         # 1-D int32 CPU
    sampling_params: SamplingParams
    images: Optional[torch.Tensor] = None   # [n, 3, S, S] uint8, resized; one block of placeholder tokens per image


@dataclass
class AbortBackendMsg(BaseMsg):
    uid: int


@dataclass
class ExitMsg(BaseMsg):
    pass


@dataclass
class BatchMsg(BaseMsg):
    data: List[BaseMsg] = field(default_factory=list)


# ---- scheduler → detokenizer ----
@dataclass
class DetokenizeMsg(BaseMsg):
    uid: int
    next_token: int
    finished: bool
    finish_reason: Optional[str] = None   # stop | length | abort | error
    logprob: Optional[float] = None
    top_logprobs: Optional[List[List[float]]] = None   # [[token_id, logprob], ...]
    error: Optional[str] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0


@dataclass
class StatsMsg(BaseMsg):
    dp_rank: int = 0
    values: Dict[str, float] = field(default_factory=dict)


# ---- detokenizer → frontend ----
@dataclass
class UserReply(BaseMsg):
    uid: int
    incremental_output: str
    finished: bool
    finish_reason: Optional[str] = None
    token_ids: List[int] = field(default_factory=list)
    logprobs: Optional[List[Dict[str, Any]]] = None
    error: Optional[str] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
