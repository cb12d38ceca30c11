"""Messages exchanged between the frontend, the tokenizer workers and the schedulers."""
from .types import (
    AbortBackendMsg, AbortMsg, BaseMsg, BatchMsg, DetokenizeMsg, ExitMsg, StatsMsg, TokenizeMsg,
    UserMsg, UserReply,
)
from .codec import decode_msg, encode_msg

__all__ = [
    "AbortBackendMsg", "AbortMsg", "BaseMsg", "BatchMsg", "DetokenizeMsg", "ExitMsg", "StatsMsg",
    "TokenizeMsg", "UserMsg", "UserReply", "decode_msg", "encode_msg",
]
