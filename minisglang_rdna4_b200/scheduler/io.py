"""Scheduler message I/O over ZMQ for a served (online) deployment
(python/minisgl/scheduler/io.py:21-217).

Rank 0 of a tensor-parallel group pulls request messages from the tokenizer, tells the other
ranks how many it got with a gloo broadcast and republishes the raw bytes on a PUB socket;
the other ranks read exactly that many from their SUB socket, so every rank processes the
same messages in the same order. Only rank 0 pushes replies to the detokenizer.
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch
import torch.distributed as dist

from ..message import BaseMsg, BatchMsg, DetokenizeMsg, StatsMsg, decode_msg
from ..utils import init_logger
from ..utils.mp import ZmqPubQueue, ZmqPullQueue, ZmqPushQueue, ZmqSubQueue

logger = init_logger(__name__)


class SchedulerIOMixin:
    """Mixed into ``Scheduler``; needs ``self.config`` and ``self.engine``."""

    def init_io(self) -> None:
        cfg = self.config
        self._tp_rank, self._tp_size = cfg.tp_rank, cfg.tp_size
        self._cpu_group = self.engine.cpu_group
        self._pull = self._pub = self._sub = self._push = None
        if self._tp_rank == 0:
            self._pull = ZmqPullQueue(cfg.zmq_backend_addr, create=True)
            self._push = ZmqPushQueue(cfg.zmq_detokenizer_addr, create=False)
            if self._tp_size > 1:
                self._pub = ZmqPubQueue(cfg.zmq_scheduler_broadcast_addr)
        else:
            self._sub = ZmqSubQueue(cfg.zmq_scheduler_broadcast_addr)
        if self._tp_size > 1:
            self._handshake()
        self._last_stats = time.monotonic()

    def _handshake(self) -> None:
        """PUB/SUB drops messages published before the subscription is live: rank 0 publishes
        probes until every rank has acknowledged one over gloo."""
        flag = torch.zeros(1, dtype=torch.int64)
        for _ in range(200):
            if self._tp_rank == 0:
                self._pub.put(BatchMsg(data=[]))
                time.sleep(0.01)
                flag.fill_(1)
            else:
                got = self._sub.get(timeout_ms=50)
                flag.fill_(1 if got is not None else 0)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self._cpu_group)
            if int(flag.item()) == 1:
                # drain extra probes
                if self._sub is not None:
                    while not self._sub.empty():
                        self._sub.get()
                dist.barrier(group=self._cpu_group)
                return
        raise RuntimeError("scheduler broadcast handshake did not complete")

    def receive_msg(self, blocking: bool) -> List[BaseMsg]:
        msgs: List[BaseMsg] = []
        if self._tp_size == 1:
            if blocking:
                first = self._pull.get(timeout_ms=100)
                if first is not None:
                    msgs.append(first)
            msgs.extend(self._pull.drain())
            return msgs
        count = torch.zeros(1, dtype=torch.int64)
        if self._tp_rank == 0:
            raws: List[bytes] = []
            if blocking and self._pull.sock.poll(20):
                raws.append(self._pull.get_raw())
            while self._pull.sock.poll(0):
                raws.append(self._pull.get_raw())
            count.fill_(len(raws))
            dist.broadcast(count, src=self.config.dp_rank * self._tp_size, group=self._cpu_group)
            for raw in raws:
                self._pub.put_raw(raw)
                msgs.append(decode_msg(raw))
        else:
            dist.broadcast(count, src=self.config.dp_rank * self._tp_size, group=self._cpu_group)
            for _ in range(int(count.item())):
                got = self._sub.get(timeout_ms=int(self.config.distributed_timeout * 1000))
                if got is None:
                    raise RuntimeError("lost a broadcast message from rank 0")
                msgs.append(got)
        return msgs

    def send_result(self, replies: List[DetokenizeMsg]) -> None:
        if self._push is not None and replies:
            self._push.put(BatchMsg(data=list(replies)))
        self._maybe_send_stats()

    def _maybe_send_stats(self) -> None:
        now = time.monotonic()
        if self._push is not None and now - self._last_stats > 1.0:
            self._last_stats = now
            self._push.put(self.stats_snapshot())
