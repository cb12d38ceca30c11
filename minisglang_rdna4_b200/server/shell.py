"""Interactive terminal chat against a running backend (``--shell-mode``;
python/minisgl/server/api_server.py:4302)."""
from __future__ import annotations

import asyncio

from ..config import ServerArgs
from ..core import SamplingParams
from ..env import ENV
from ..message import TokenizeMsg, UserReply
from ..utils.mp import ZmqAsyncPullQueue, ZmqAsyncPushQueue


async def _chat(args: ServerArgs) -> None:
    send = ZmqAsyncPushQueue(args.zmq_tokenizer_addr, create=False)
    recv = ZmqAsyncPullQueue(args.zmq_frontend_addr, create=True)
    history = []
    if ENV.SHELL_SYSTEM_PROMPT.value:
        history.append({"role": "system", "content": ENV.SHELL_SYSTEM_PROMPT.value})
    uid = 0
    loop = asyncio.get_event_loop()
    while True:
        try:
            line = await loop.run_in_executor(None, input, "> ")
        except (EOFError, KeyboardInterrupt):
            return
        if line.strip() in ("/exit", "/quit"):
            return
        if line.strip() == "/reset":
            history = history[:1] if history and history[0]["role"] == "system" else []
            continue
        history.append({"role": "user", "content": line})
        uid += 1
        await send.put(TokenizeMsg(uid, history, SamplingParams(temperature=0.6, top_p=0.95, max_tokens=2048)))
        text = []
        while True:
            msg = await recv.get()
            if not isinstance(msg, UserReply) or msg.uid != uid:
                continue
            print(msg.incremental_output, end="", flush=True)
            text.append(msg.incremental_output)
            if msg.finished:
                print()
                break
        history.append({"role": "assistant", "content": "".join(text)})


def run_shell(args: ServerArgs) -> None:
    asyncio.run(_chat(args))
