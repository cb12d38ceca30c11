"""Stand-alone recursive-self-aggregation proxy (python/minisgl/rsa/server.py:49): an OpenAI-compatible
endpoint that sits in front of ANY chat-completions server, fans a request out into N rollouts and
T - 1 aggregation rounds against it, and answers with the selected result. Requests without
``rsa`` (and without an effort the ladder maps) are forwarded unchanged.

``python -m minisglang_rdna4_b200.rsa.proxy --upstream http://127.0.0.1:1919 --port 1920 --rsa-n 4``
"""
from __future__ import annotations

import argparse
import time
import uuid
from dataclasses import fields, replace
from typing import Any, Awaitable, Callable, Dict, Optional

from .core import RSAParams, run_rsa

Post = Callable[[str, Dict[str, Any]], Awaitable[Dict[str, Any]]]


def params_for(body: Dict[str, Any], defaults: RSAParams, effort_ladder: bool) -> Optional[RSAParams]:
    rsa = body.get("rsa")
    if rsa:
        if isinstance(rsa, dict):
            allowed = {f.name for f in fields(RSAParams)}
            bad = sorted(set(rsa) - allowed)
            if bad:
                raise ValueError(f"unknown rsa fields: {bad}")
            return replace(defaults, **rsa)
        return defaults
    if effort_ladder and body.get("reasoning_effort"):
        return RSAParams.from_effort(body["reasoning_effort"])
    return None


async def handle_chat(body: Dict[str, Any], post: Post, defaults: RSAParams, effort_ladder: bool = False
                      ) -> Dict[str, Any]:
    """One ``/v1/chat/completions`` request body in, one response object out."""
    params = params_for(body, defaults, effort_ladder)
    if params is None:
        return await post("/v1/chat/completions", body)
    passthrough = {k: v for k, v in body.items()
                   if k in ("model", "chat_template_kwargs", "enable_thinking", "stop", "seed")}
    usage = {"prompt_tokens": 0, "completion_tokens": 0}

    async def generate(msgs, max_tokens, temperature, top_p) -> str:
        out = await post("/v1/chat/completions", {**passthrough, "messages": msgs, "max_tokens": int(max_tokens),
                                                  "temperature": float(temperature), "top_p": float(top_p),
                                                  "stream": False})
        u = out.get("usage") or {}
        usage["prompt_tokens"] += int(u.get("prompt_tokens", 0))
        usage["completion_tokens"] += int(u.get("completion_tokens", 0))
        return (out["choices"][0]["message"].get("content") or "") if out.get("choices") else ""

    result = await run_rsa(list(body.get("messages") or []), params, generate)
    usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
    return {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()),
            "model": body.get("model") or "rsa",
            "choices": [{"index": 0, "message": {"role": "assistant", "content": result["answer"]},
                         "finish_reason": "stop"}],
            "usage": usage,
            "rsa": {"rounds": result["rounds"], "calls": result["calls"], "n": params.n, "k": params.k, "t": params.t}}


def create_proxy_app(upstream: str, defaults: RSAParams, effort_ladder: bool = False, timeout_s: float = 600.0):
    import aiohttp
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse

    app = FastAPI(title="rsa proxy")

    async def post(path: str, payload: Dict[str, Any]) -> Dict[str, Any]:
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=timeout_s)) as session:
            async with session.post(upstream.rstrip("/") + path, json=payload) as resp:
                if resp.status != 200:
                    raise HTTPException(status_code=resp.status, detail=(await resp.text())[:500])
                return await resp.json()

    @app.get("/health")
    async def health():
        return {"status": "ok", "upstream": upstream}

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        body = await request.json()
        if body.get("stream") and params_for(body, defaults, effort_ladder) is not None:
            raise HTTPException(status_code=400, detail="the rsa proxy answers aggregated requests without streaming")
        try:
            return JSONResponse(await handle_chat(body, post, defaults, effort_ladder))
        except ValueError as exc:
            raise HTTPException(status_code=400, detail=str(exc))

    return app


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--upstream", required=True)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=1920)
    ap.add_argument("--rsa-n", type=int, default=4)
    ap.add_argument("--rsa-k", type=int, default=2)
    ap.add_argument("--rsa-t", type=int, default=2)
    ap.add_argument("--rsa-max-tokens", type=int, default=1024)
    ap.add_argument("--rsa-agg-max-tokens", type=int, default=1024)
    ap.add_argument("--rsa-temperature", type=float, default=0.7)
    ap.add_argument("--rsa-top-p", type=float, default=0.95)
    ap.add_argument("--rsa-selection", default="vote", choices=["vote", "first", "longest"])
    ap.add_argument("--rsa-max-concurrency", type=int, default=8)
    ap.add_argument("--rsa-request-timeout", type=float, default=600.0)
    ap.add_argument("--rsa-effort-ladder", action="store_true")
    a = ap.parse_args(argv)
    import uvicorn

    defaults = RSAParams(n=a.rsa_n, k=a.rsa_k, t=a.rsa_t, max_tokens=a.rsa_max_tokens,
                         agg_max_tokens=a.rsa_agg_max_tokens, temperature=a.rsa_temperature, top_p=a.rsa_top_p,
                         selection=a.rsa_selection, max_concurrency=a.rsa_max_concurrency)
    uvicorn.run(create_proxy_app(a.upstream, defaults, a.rsa_effort_ladder, a.rsa_request_timeout),
                host=a.host, port=a.port, log_level="warning")


if __name__ == "__main__":
    main()
