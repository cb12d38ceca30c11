"""Tokenizer / detokenizer worker process (python/minisgl/tokenizer/server.py:50-268).

One loop serves both directions: ``TokenizeMsg`` from the frontend becomes a ``UserMsg`` for
a scheduler replica (round-robin over data-parallel replicas), ``DetokenizeMsg`` batches from
the schedulers become ``UserReply`` text deltas for the frontend. A stop string hit ends the
request: the worker tells every replica to abort it. ``StatsMsg`` is relayed unchanged.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import ServerArgs
from ..message import (
    AbortBackendMsg, AbortMsg, BatchMsg, DetokenizeMsg, ExitMsg, StatsMsg, TokenizeMsg, UserMsg, UserReply,
)
from ..utils import init_logger
from ..utils.mp import ZmqPullQueue, ZmqPushQueue
from .detokenize import DetokenizeManager
from .simple import load_tokenizer
from .tokenize import TokenizeManager

logger = init_logger(__name__)


class TokenizerWorker:
    def __init__(self, args: ServerArgs, tokenizer=None) -> None:
        self.args = args
        self.tokenizer = tokenizer or load_tokenizer(args.model_path)
        self.tok = TokenizeManager(self.tokenizer, args.chat_template, args.chat_template_kwargs)
        self.detok = DetokenizeManager(self.tokenizer)
        self.next_replica = 0
        self.route: Dict[int, int] = {}
        self.logprob_n: Dict[int, int] = {}

    # ---- pure handlers (unit-testable without sockets) ----
    def on_tokenize(self, msg: TokenizeMsg):
        """Returns ``(replica, UserMsg)`` or ``(None, UserReply)`` when the prompt is invalid."""
        try:
            ids = self.tok.tokenize(msg.text, msg.chat_template_kwargs, msg.tools, msg.add_generation_prompt)
        except Exception as exc:
            return None, UserReply(msg.uid, "", True, "error", error=str(exc))
        pixels = None
        if getattr(msg, "images", None):
            try:
                pre = self._vision()
                pixels = pre.batch(msg.images)
                ids = torch.tensor(pre.expand_placeholders(ids.tolist(), len(msg.images)), dtype=torch.int32)
            except Exception as exc:
                return None, UserReply(msg.uid, "", True, "error", error=f"image input: {exc}")
        sp = msg.sampling_params
        self.detok.register(msg.uid, sp.stop, sp.stop_keep)
        replica = self.next_replica
        self.next_replica = (self.next_replica + 1) % max(self.args.dp_size, 1)
        self.route[msg.uid] = replica
        self.logprob_n[msg.uid] = sp.logprobs
        return replica, UserMsg(msg.uid, ids, sp, images=pixels)

    def _vision(self):
        """Image preprocessor of the served checkpoint (built on the first request with an image)."""
        pre = getattr(self, "_vision_pre", None)
        if pre is None:
            from ..models.config import ModelConfig
            from .vision import VisionPreprocessor

            vc = ModelConfig.from_hf(self.args.model_path).vision
            if vc is None:
                raise ValueError("this model takes no image input")
            pre = self._vision_pre = VisionPreprocessor.from_vision_config(vc)
        return pre

    def on_detokenize(self, msg: DetokenizeMsg):
        """Returns ``(UserReply or None, abort uid or None)``."""
        if msg.error is not None:
            self._forget(msg.uid)
            return UserReply(msg.uid, "", True, "error", error=msg.error), None
        if msg.uid not in self.detok.states:
            return None, None  # already finished by a stop string
        text, hit, _which = self.detok.step(msg.uid, msg.next_token, msg.finished)
        finished = msg.finished or hit
        reason = "stop" if hit else msg.finish_reason
        logprobs = None
        if msg.logprob is not None:
            top = [{"token_id": int(t), "token": self.tokenizer.decode([int(t)]), "logprob": float(lp)}
                   for t, lp in (msg.top_logprobs or [])]
            logprobs = [{"token_id": msg.next_token, "token": self.tokenizer.decode([msg.next_token]),
                         "logprob": msg.logprob, "top": top}]
        reply = UserReply(msg.uid, text, finished, reason if finished else None, [msg.next_token], logprobs,
                          prompt_tokens=msg.prompt_tokens, cached_tokens=msg.cached_tokens)
        abort = msg.uid if hit and not msg.finished else None
        if finished:
            self._forget(msg.uid)
        return reply, abort

    def _forget(self, uid: int) -> None:
        self.detok.finish(uid)
        self.route.pop(uid, None)
        self.logprob_n.pop(uid, None)


def tokenize_worker(args: ServerArgs, ready=None, tokenizer=None) -> None:
    """Process entry point."""
    worker = TokenizerWorker(args, tokenizer)
    pull_front = ZmqPullQueue(args.zmq_tokenizer_addr, create=True)
    pull_back = ZmqPullQueue(args.zmq_detokenizer_addr, create=True)
    push_front = ZmqPushQueue(args.zmq_frontend_addr, create=False)
    push_back = [ZmqPushQueue(args.backend_addr_of(r), create=False) for r in range(max(args.dp_size, 1))]
    if ready is not None:
        ready.put("tokenizer ready")
    import zmq

    poller = zmq.Poller()
    poller.register(pull_front.sock, zmq.POLLIN)
    poller.register(pull_back.sock, zmq.POLLIN)
    running = True
    while running:
        events = dict(poller.poll(100))
        if pull_front.sock in events:
            for msg in pull_front.drain():
                if isinstance(msg, TokenizeMsg):
                    replica, out = worker.on_tokenize(msg)
                    if replica is None:
                        push_front.put(out)
                    else:
                        push_back[replica].put(out)
                elif isinstance(msg, AbortMsg):
                    worker._forget(msg.uid)
                    for q in push_back:  # aborts fan out to every replica
                        q.put(AbortBackendMsg(msg.uid))
                elif isinstance(msg, ExitMsg):
                    for q in push_back:
                        q.put(ExitMsg())
                    running = False
        if pull_back.sock in events:
            for msg in pull_back.drain():
                items = msg.data if isinstance(msg, BatchMsg) else [msg]
                for item in items:
                    if isinstance(item, StatsMsg):
                        push_front.put(item)
                    elif isinstance(item, DetokenizeMsg):
                        reply, abort = worker.on_detokenize(item)
                        if reply is not None:
                            push_front.put(reply)
                        if abort is not None:
                            for q in push_back:
                                q.put(AbortBackendMsg(abort))
