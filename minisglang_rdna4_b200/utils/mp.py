"""ZMQ queues carrying msgpack-encoded messages between the frontend, the tokenizer workers
and the schedulers (python/minisgl/utils/mp.py:12-154): PUSH/PULL for point-to-point links,
PUB/SUB for the rank-0 → other-ranks fan-out."""
from __future__ import annotations

from typing import Any, Callable, Generic, List, Optional, TypeVar

import zmq
import zmq.asyncio

from ..message.codec import decode_msg, encode_msg

T = TypeVar("T")


class ZmqPushQueue(Generic[T]):
    def __init__(self, addr: str, create: bool) -> None:
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.PUSH)
        self.sock.setsockopt(zmq.LINGER, 0)
        (self.sock.bind if create else self.sock.connect)(addr)

    def put(self, obj: T) -> None:
        self.sock.send(encode_msg(obj), copy=False)

    def stop(self) -> None:
        self.sock.close()


class ZmqPullQueue(Generic[T]):
    def __init__(self, addr: str, create: bool) -> None:
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.PULL)
        self.sock.setsockopt(zmq.LINGER, 0)
        (self.sock.bind if create else self.sock.connect)(addr)

    def get(self, timeout_ms: Optional[int] = None) -> Optional[T]:
        if timeout_ms is not None and not self.sock.poll(timeout_ms):
            return None
        return decode_msg(self.sock.recv())

    def get_raw(self) -> bytes:
        return self.sock.recv()

    def empty(self) -> bool:
        return self.sock.poll(0) == 0

    def drain(self) -> List[T]:
        out: List[T] = []
        while self.sock.poll(0):
            out.append(decode_msg(self.sock.recv()))
        return out

    def stop(self) -> None:
        self.sock.close()


class ZmqAsyncPushQueue(Generic[T]):
    def __init__(self, addr: str, create: bool) -> None:
        self.ctx = zmq.asyncio.Context.instance()
        self.sock = self.ctx.socket(zmq.PUSH)
        self.sock.setsockopt(zmq.LINGER, 0)
        (self.sock.bind if create else self.sock.connect)(addr)

    async def put(self, obj: T) -> None:
        await self.sock.send(encode_msg(obj), copy=False)

    def stop(self) -> None:
        self.sock.close()


class ZmqAsyncPullQueue(Generic[T]):
    def __init__(self, addr: str, create: bool) -> None:
        self.ctx = zmq.asyncio.Context.instance()
        self.sock = self.ctx.socket(zmq.PULL)
        self.sock.setsockopt(zmq.LINGER, 0)
        (self.sock.bind if create else self.sock.connect)(addr)

    async def get(self) -> T:
        return decode_msg(await self.sock.recv())

    def stop(self) -> None:
        self.sock.close()


class ZmqPubQueue(Generic[T]):
    def __init__(self, addr: str) -> None:
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.PUB)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.bind(addr)

    def put_raw(self, raw: bytes) -> None:
        self.sock.send(raw, copy=False)

    def put(self, obj: T) -> None:
        self.sock.send(encode_msg(obj), copy=False)

    def stop(self) -> None:
        self.sock.close()


class ZmqSubQueue(Generic[T]):
    def __init__(self, addr: str) -> None:
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.SUB)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.setsockopt(zmq.SUBSCRIBE, b"")
        self.sock.connect(addr)

    def get(self, timeout_ms: Optional[int] = None) -> Optional[T]:
        if timeout_ms is not None and not self.sock.poll(timeout_ms):
            return None
        return decode_msg(self.sock.recv())

    def empty(self) -> bool:
        return self.sock.poll(0) == 0

    def stop(self) -> None:
        self.sock.close()
