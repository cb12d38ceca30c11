"""OpenAI-compatible HTTP frontend (python/minisgl/server/api_server.py): ``/generate``,
``/v1/chat/completions``, ``/v1/completions``, ``/v1/models``, ``/health``, ``/metrics``.

The frontend owns no model state. It turns a request into a ``TokenizeMsg`` for the tokenizer
worker, then demultiplexes ``UserReply`` text deltas into per-request queues and renders them
as JSON or server-sent events. A client that disconnects mid-stream aborts its request.
"""
from __future__ import annotations

import os

import asyncio
import json
import time
import uuid
from dataclasses import replace
from typing import Any, AsyncIterator, Dict, List, Optional, Union

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse
from pydantic import BaseModel, Field, model_validator

from ..config import ServerArgs
from ..core import SamplingParams
from ..env import ENV
from ..message import AbortMsg, StatsMsg, TokenizeMsg, UserReply
from ..utils import init_logger
from .metrics import FrontendMetrics
from .reasoning import ReasoningParser, ReasoningStreamState, resolve_reasoning_parser
from .tools import (ToolCallStreamState, grammar_from_tools, parse_tool_calls, resolve_tool_format,
                    structural_tag_for_tools, tool_openers_closers)

logger = init_logger(__name__)


# ------------------------------------------------------------------------------------------ schemas
class GenerateRequest(BaseModel):
    prompt: str
    max_tokens: int = Field(default_factory=lambda: ENV.DEFAULT_MAX_TOKENS.value)
    ignore_eos: bool = False
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None
    cam_read: Optional[bool] = None
    cam_write: Optional[bool] = None


class ChatMessage(BaseModel):
    role: str
    content: Union[str, List[Dict[str, Any]], None] = None
    name: Optional[str] = None
    tool_calls: Optional[List[Dict[str, Any]]] = None
    tool_call_id: Optional[str] = None
    reasoning_content: Optional[str] = None


def extract_images(messages: List[Dict[str, Any]]) -> List[bytes]:
    """Encoded image files of a chat request, in prompt order. OpenAI ``image_url`` parts (``data:``
    URLs only: this server fetches nothing) and ``{"type": "image", "image": <data URL>}`` parts are
    rewritten in place to bare ``{"type": "image"}`` parts, which is what chat templates render as
    the begin-of-image marker (python/minisgl/tokenizer/vision.py:92-140)."""
    import base64

    out: List[bytes] = []
    for m in messages:
        parts = m.get("content")
        if not isinstance(parts, list):
            continue
        for i, part in enumerate(parts):
            kind = part.get("type")
            url = None
            if kind == "image_url":
                url = (part.get("image_url") or {}).get("url") if isinstance(part.get("image_url"), dict) else part.get(
                    "image_url")
            elif kind == "image" and isinstance(part.get("image"), str):
                url = part["image"]
            if url is None:
                continue
            if not str(url).startswith("data:") or "," not in url:
                raise RequestRejected("images are accepted as data: URLs only (this server fetches nothing)", "messages",
                                      "invalid_image_url")
            try:
                out.append(base64.b64decode(url.split(",", 1)[1], validate=False))
            except Exception:
                raise RequestRejected("an image part does not hold base64 data", "messages", "invalid_image_url")
            parts[i] = {"type": "image"}
    return out


class RequestRejected(ValueError):
    """A request field this server cannot honour: answered with 400 and the OpenAI error object
    ``{"error": {message, type, param, code}}`` (python/minisgl/server/api_server.py:1473-1590)."""

    def __init__(self, message: str, param: Optional[str] = None, code: str = "unsupported_parameter") -> None:
        super().__init__(message)
        self.param, self.code = param, code


def error_body(message: str, param: Optional[str] = None, code: Optional[str] = None, detail=None) -> Dict[str, Any]:
    body = {"error": {"message": message, "type": "invalid_request_error", "param": param, "code": code}}
    body["detail"] = detail if detail is not None else message
    return body


def reject_unclosed_tool_call(messages, fmt: Optional[str]) -> Optional[RequestRejected]:
    """A final assistant turn that ends inside a very large unclosed tool-call block is a
    length-truncated call sent back for continuation; the model resumes the runaway and every retry
    burns another full budget. Small truncated calls (the model can still close them) and prose that
    merely quotes an opener pass (python/minisgl/server/api_server.py:1506-1541)."""
    limit = ENV.TOOLCALL_CONT_LIMIT.value
    if limit <= 0 or not messages:
        return None
    last = messages[-1]
    if last.role != "assistant" or not isinstance(last.content, str) or len(last.content) < limit:
        return None
    scan = ToolCallStreamState(fmt=fmt)
    scan.push(last.content)
    if scan.in_call is None or scan.held_chars < limit:
        return None
    return RequestRejected(
        f"the final assistant message ends inside an unclosed tool-call block: {scan.held_chars} characters follow "
        f"the last {scan.in_call[0]!r} with no closer. A block this large cannot be completed by continuation; "
        "drop the partial call (or raise max_tokens on the original request) instead of re-sending it.",
        "messages", "unclosed_tool_call")


class OpenAICompletionRequest(BaseModel):
    model: Optional[str] = None
    prompt: Union[str, List[int], None] = None
    messages: Optional[List[ChatMessage]] = None
    max_tokens: Optional[int] = None
    max_completion_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    min_p: Optional[float] = None
    n: int = 1
    stream: bool = False
    stream_options: Optional[Dict[str, Any]] = None
    stop: Union[str, List[str], None] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    response_format: Optional[Dict[str, Any]] = None
    ignore_eos: bool = False
    tools: Optional[List[Dict[str, Any]]] = None
    tool_choice: Any = None
    chat_template_kwargs: Optional[Dict[str, Any]] = None
    enable_thinking: Optional[bool] = None
    reasoning_max_tokens: Optional[int] = None
    reasoning_effort: Optional[str] = None
    # recursive self-aggregation: true = the server's defaults, or an object overriding n / k / t / ...
    # the same three knobs in the shapes other APIs use: ``reasoning: {effort, max_tokens, enabled}``
    # and ``thinking: true | {type: "enabled" | "disabled", budget_tokens}``; folded into the fields above
    reasoning: Optional[Dict[str, Any]] = None
    thinking: Union[bool, Dict[str, Any], None] = None
    rsa: Union[bool, Dict[str, Any], None] = None
    # associative memory: per-request override of the ambient read / write defaults (MSGL_CAM_AUTO,
    # MSGL_CAM_AUTO_WRITE); only meaningful when the server runs with MSGL_CAM=1
    cam_read: Optional[bool] = None
    cam_write: Optional[bool] = None
    logprobs: Union[bool, int, None] = None
    top_logprobs: Optional[int] = None
    seed: Optional[int] = None
    # accepted and ignored
    user: Optional[str] = None
    store: Optional[bool] = None
    metadata: Optional[Dict[str, Any]] = None
    service_tier: Optional[str] = None
    parallel_tool_calls: Optional[bool] = None
    # rejected when set to something the engine cannot honour
    logit_bias: Optional[Dict[str, float]] = None
    echo: Optional[bool] = None
    suffix: Optional[str] = None
    best_of: Optional[int] = None

    @model_validator(mode="after")
    def _check(self):
        if self.messages is None and self.prompt is None:
            raise RequestRejected("either `messages` or `prompt` is required", "messages", "missing_required_parameter")
        mt = self.max_completion_tokens if self.max_completion_tokens is not None else self.max_tokens
        if mt is not None and mt < 1:
            raise RequestRejected("max_tokens must be at least 1", "max_tokens", "invalid_value")
        if self.n != 1:
            raise RequestRejected(f"n={self.n} is not supported: this server returns a single choice; send n requests", "n")
        if self.logit_bias:
            raise RequestRejected("logit_bias is not supported by this server", "logit_bias")
        if self.echo:
            raise RequestRejected("echo is not supported: this server returns the completion only", "echo")
        if self.suffix:
            raise RequestRejected("suffix (fill-in-the-middle) is not supported by this server", "suffix")
        if self.best_of not in (None, 1):
            raise RequestRejected(f"best_of={self.best_of} is not supported: this server samples a single completion", "best_of")
        if isinstance(self.reasoning, dict):
            r = self.reasoning
            if self.reasoning_effort is None and isinstance(r.get("effort"), str):
                self.reasoning_effort = r["effort"]
            if self.reasoning_max_tokens is None and isinstance(r.get("max_tokens"), int):
                self.reasoning_max_tokens = r["max_tokens"]
            if self.enable_thinking is None and isinstance(r.get("enabled"), bool):
                self.enable_thinking = r["enabled"]
        if self.thinking is not None:
            t = self.thinking
            if isinstance(t, bool):
                on, budget = t, None
            else:
                on = {"enabled": True, "disabled": False}.get(str(t.get("type", "")).lower())
                budget = t.get("budget_tokens")
                if on is None and "type" in t:
                    raise RequestRejected("thinking.type must be `enabled` or `disabled`", "thinking", "invalid_value")
            if self.enable_thinking is None and on is not None:
                self.enable_thinking = on
            if self.reasoning_max_tokens is None and isinstance(budget, int) and budget > 0:
                self.reasoning_max_tokens = budget
        return self

    def resolved_max_tokens(self) -> int:
        mt = self.max_completion_tokens if self.max_completion_tokens is not None else self.max_tokens
        return int(mt) if mt is not None else ENV.DEFAULT_MAX_TOKENS.value


# ------------------------------------------------------------------------------------------ frontend
class FrontendManager:
    """Owns the ZMQ links of the frontend and the per-request reply queues."""

    def __init__(self, args: ServerArgs, send_queue=None, recv_queue=None) -> None:
        self.args = args
        self.send_queue = send_queue
        self.recv_queue = recv_queue
        self.queues: Dict[int, asyncio.Queue] = {}
        self.uid = 0
        self.metrics = FrontendMetrics(args.model_name)
        self._listener: Optional[asyncio.Task] = None

    def new_user(self) -> int:
        self.uid += 1
        self.queues[self.uid] = asyncio.Queue()
        self.metrics.on_request(self.uid)
        return self.uid

    async def send_one(self, msg) -> None:
        await self.send_queue.put(msg)

    async def listen(self) -> None:
        while True:
            msg = await self.recv_queue.get()
            if isinstance(msg, StatsMsg):
                self.metrics.on_scheduler_stats(msg.dp_rank, msg.values)
            elif isinstance(msg, UserReply):
                q = self.queues.get(msg.uid)
                if q is not None:
                    q.put_nowait(msg)

    def ensure_listener(self) -> None:
        if self._listener is None and self.recv_queue is not None:
            self._listener = asyncio.get_event_loop().create_task(self.listen())

    async def replies(self, uid: int) -> AsyncIterator[UserReply]:
        q = self.queues[uid]
        try:
            while True:
                msg: UserReply = await q.get()
                self.metrics.on_token(uid, len(msg.token_ids) or 1)
                yield msg
                if msg.finished:
                    self.metrics.on_finish(uid, msg.finish_reason, msg.prompt_tokens, msg.cached_tokens)
                    return
        finally:
            self.queues.pop(uid, None)

    async def abort_user(self, uid: int) -> None:
        if uid in self.queues:
            self.queues.pop(uid, None)
            self.metrics.on_finish(uid, "abort")
            await self.send_one(AbortMsg(uid))


# ------------------------------------------------------------------------------------------ helpers
# The served model's recommended sampling (generation_config.json), applied to the fields a
# request leaves unset; filled by ``set_sampling_defaults`` when the server starts
# (python/minisgl/utils/hf.py:192: a repack served with top_p = 1 / top_k = -1 while its card says
# 0.95 / 64 samples from the whole distribution).
_SAMPLING_DEFAULTS: Dict[str, float] = {}


def set_sampling_defaults(model_path: str) -> Dict[str, float]:
    from ..utils.hf import sampling_defaults

    _SAMPLING_DEFAULTS.clear()
    _SAMPLING_DEFAULTS.update(sampling_defaults(model_path))
    return dict(_SAMPLING_DEFAULTS)


def sampling_from_request(req: OpenAICompletionRequest, reasoning: Optional[ReasoningParser],
                          chat_template: Optional[str]) -> SamplingParams:
    stop = [req.stop] if isinstance(req.stop, str) else list(req.stop or [])
    logprobs = 0
    if req.logprobs:
        logprobs = int(req.top_logprobs or (req.logprobs if isinstance(req.logprobs, int) and not isinstance(req.logprobs, bool) else 1))
        logprobs = max(1, min(logprobs, 20))
    grammar, required = None, False
    if req.response_format:
        kind = req.response_format.get("type")
        if kind == "json_object":
            grammar, required = "json", True
        elif kind == "json_schema":
            schema = (req.response_format.get("json_schema") or {}).get("schema") or req.response_format.get("schema")
            grammar, required = json.dumps(schema or {}), True
        elif kind not in (None, "text"):
            raise ValueError(f"unsupported response_format type {kind!r}")
    openers: List[str] = []
    closers: List[str] = []
    if req.tools and req.tool_choice != "none":
        fmt = resolve_tool_format(None, chat_template)
        forced = grammar_from_tools(req.tools, req.tool_choice, fmt)
        if forced is not None and grammar is None:
            grammar, required = forced, True
        elif grammar is None and os.environ.get("MSGL_TOOL_AUTO_CONSTRAIN", "0") == "1":
            grammar = structural_tag_for_tools(req.tools, fmt)     # free text, schema-checked call bodies
        openers, closers = tool_openers_closers(chat_template, fmt)
    thinking = req.enable_thinking
    if thinking is None and req.chat_template_kwargs:
        thinking = req.chat_template_kwargs.get("enable_thinking")
    sp = SamplingParams(
        temperature=float(_SAMPLING_DEFAULTS.get("temperature", 0.0)) if req.temperature is None else float(req.temperature),
        top_k=int(_SAMPLING_DEFAULTS.get("top_k", -1)) if req.top_k is None else int(req.top_k),
        top_p=float(_SAMPLING_DEFAULTS.get("top_p", 1.0)) if req.top_p is None else float(req.top_p),
        min_p=float(_SAMPLING_DEFAULTS.get("min_p", 0.0)) if req.min_p is None else float(req.min_p),
        ignore_eos=req.ignore_eos, max_tokens=req.resolved_max_tokens(), logprobs=logprobs,
        presence_penalty=req.presence_penalty, frequency_penalty=req.frequency_penalty, stop=stop,
        grammar=grammar, grammar_required=required, seed=req.seed,
        tool_call_openers=openers, tool_call_closers=closers,
    )
    if reasoning is not None and thinking is not False:
        sp = replace(sp, think_close_delim=reasoning.close, think_span_open=reasoning.starts_open,
                     think_budget=int(req.reasoning_max_tokens or 0), think_tool_release=list(openers),
                     think_answer_delim=reasoning.answer_delim, think_close_prefix=reasoning.close_prefix,
                     think_close_suffix=reasoning.close_suffix)
    return sp


def _sse(obj: Any) -> str:
    return "data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n"


def _usage(prompt: int, completion: int, cached: int) -> Dict[str, Any]:
    return {"prompt_tokens": prompt, "completion_tokens": completion, "total_tokens": prompt + completion,
            "prompt_tokens_details": {"cached_tokens": cached}}


async def stream_with_cancellation(request: Request, gen: AsyncIterator[str], on_cancel) -> AsyncIterator[str]:
    """Forward ``gen`` while polling the connection; a vanished client triggers ``on_cancel``."""
    try:
        async for chunk in gen:
            if await request.is_disconnected():
                await on_cancel()
                return
            yield chunk
    except asyncio.CancelledError:
        await on_cancel()
        raise


# ------------------------------------------------------------------------------------------ app
# ------------------------------------------------------------------------------------------ CAM hooks
_FACT_RE = None


def looks_like_fact_statement(text: str) -> bool:
    """Does the text plausibly assert a durable fact? Questions and texts without a copula do not
    (python/minisgl/server/api_server.py:2003-2014); keeps chit-chat out of the store."""
    import re

    t = (text or "").strip()
    return bool(t) and not t.endswith("?") and re.search(r"\b(is|was|are|were)\b", t, re.IGNORECASE) is not None


def extract_facts(text: str) -> List[tuple]:
    """``(subject, relation, object)`` triples of the plain ``<subject> is|was|are|were <object>``
    sentences of the text. The reference asks the served model to extract them; this build uses
    the sentence pattern, which is deterministic and needs no extra generation."""
    import re

    out = []
    for sent in re.split(r"(?<=[.!;])\s+|\n+", text or ""):
        sent = sent.strip().rstrip(".!;")
        m = re.match(r"^(?P<s>[^,:?]{2,80}?)\s+(?P<r>is|was|are|were)\s+(?P<o>[^?]{1,200})$", sent, re.IGNORECASE)
        if m and not sent.endswith("?"):
            subj = re.sub(r"^(remember that|note that|fyi,?)\s+", "", m.group("s").strip(), flags=re.IGNORECASE)
            out.append((subj, m.group("r").lower(), m.group("o").strip()))
    return out


def cam_auto_read(memory, payload: Any, override: Optional[bool], namespace: str = "default") -> Any:
    """Transparent read: facts that match the request are stated in front of it (a system message
    for chat, a preface for a raw prompt). Unchanged when off or when nothing matches."""
    enabled = override if override is not None else os.environ.get("MSGL_CAM_AUTO", "0") == "1"
    if memory is None or not enabled:
        return payload
    if isinstance(payload, list):
        query = " ".join(str(m.get("content") or "") for m in payload if m.get("role") in ("user", "system"))
        hits = memory.lookup(query, namespace) if query.strip() else []
        if not hits:
            return payload
        note = "Known facts:\n" + "\n".join(f"- {f.subject}: {f.prompt} {f.object}".replace("  ", " ") for _, f in hits)
        return [{"role": "system", "content": note}] + list(payload)
    return memory.augment(str(payload), namespace)


def cam_auto_write(memory, text: str, override: Optional[bool], namespace: str = "default") -> int:
    """Ambient write: durable facts asserted in the latest user turn are remembered. Returns how many."""
    enabled = override if override is not None else os.environ.get("MSGL_CAM_AUTO_WRITE", "0") == "1"
    if memory is None or not enabled or not looks_like_fact_statement(text):
        return 0
    n = 0
    for subj, rel, obj in extract_facts(text):
        memory.remember(subj, rel, obj, namespace)
        n += 1
    return n


def create_app(args: ServerArgs, manager: Optional[FrontendManager] = None, chat_template: Optional[str] = None,
               tokenizer=None) -> FastAPI:
    app = FastAPI(title="minisglang-rdna4 b200")
    state = manager or FrontendManager(args)
    app.state.manager = state
    reasoning = resolve_reasoning_parser(args.reasoning_parser, chat_template, tokenizer)
    if reasoning is not None:
        logger.info("reasoning delimiters %r .. %r (%s)", reasoning.open, reasoning.close, reasoning.how or "named")
    if tokenizer is not None:
        resolve_tool_format(tokenizer, chat_template)            # log the derived tool-call format once
    created = int(time.time())

    from fastapi.exceptions import RequestValidationError

    @app.exception_handler(RequestValidationError)
    async def _invalid(request: Request, exc: RequestValidationError):
        # one OpenAI-shaped error for a body that does not validate; the first problem names the field
        errs = exc.errors()
        first = errs[0] if errs else {}
        cause = (first.get("ctx") or {}).get("error")
        if isinstance(cause, RequestRejected):
            msg, param, code = str(cause), cause.param, cause.code
        else:
            loc = [str(x) for x in first.get("loc", ()) if x != "body"]
            msg, param, code = first.get("msg", "invalid request"), (".".join(loc) or None), "invalid_value"
        detail = [{k: (str(v) if k == "ctx" else v) for k, v in e.items() if k != "input"} for e in errs]
        return JSONResponse(status_code=400, content=error_body(msg, param, code, detail))

    @app.exception_handler(HTTPException)
    async def _http_error(request: Request, exc: HTTPException):
        msg = exc.detail if isinstance(exc.detail, str) else json.dumps(exc.detail)
        return JSONResponse(status_code=exc.status_code, content=error_body(msg, None, None, exc.detail),
                            headers=getattr(exc, "headers", None))

    @app.on_event("startup")
    async def _startup() -> None:  # pragma: no cover - needs a running loop with sockets
        state.ensure_listener()

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1")
    async def v1_root():
        return {"status": "ok", "model": args.model_name}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": args.model_name, "object": "model", "created": created,
                                            "owned_by": "minisglang_rdna4_b200"}]}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(state.metrics.render(), media_type="text/plain; version=0.0.4")

    @app.post("/generate")
    async def generate(req: GenerateRequest, request: Request):
        state.ensure_listener()
        uid = state.new_user()
        sp = SamplingParams(temperature=req.temperature, top_k=req.top_k, top_p=req.top_p, min_p=req.min_p,
                            ignore_eos=req.ignore_eos, max_tokens=req.max_tokens, seed=req.seed,
                            presence_penalty=req.presence_penalty, frequency_penalty=req.frequency_penalty)
        prompt = req.prompt
        cam = getattr(app.state, "cam", None)
        if cam is not None:
            ns = request.headers.get("x-cam-namespace") or "default"
            cam_auto_write(cam, prompt, req.cam_write, ns)
            prompt = cam_auto_read(cam, prompt, req.cam_read, ns)
        await state.send_one(TokenizeMsg(uid, prompt, sp))

        async def gen():
            async for reply in state.replies(uid):
                if reply.error:
                    yield _sse({"error": reply.error})
                    break
                if reply.incremental_output:
                    yield _sse(reply.incremental_output)
            yield _sse("[DONE]")

        return StreamingResponse(stream_with_cancellation(request, gen(), lambda: state.abort_user(uid)),
                                 media_type="text/event-stream")

    async def _run(req: OpenAICompletionRequest, request: Request, chat: bool):
        state.ensure_listener()
        try:
            sp = sampling_from_request(req, reasoning if chat else None, chat_template)
        except ValueError as exc:
            raise HTTPException(status_code=400, detail=str(exc))
        uid = state.new_user()
        if chat:
            if req.messages is None:
                raise HTTPException(status_code=400, detail="`messages` is required")
            payload: Any = [m.model_dump(exclude_none=True) for m in req.messages]
        else:
            payload = req.prompt if req.prompt is not None else [m.model_dump(exclude_none=True) for m in req.messages]
        images: List[bytes] = []
        if chat:
            try:
                images = extract_images(payload)
            except RequestRejected as bad:
                state.queues.pop(uid, None)
                return JSONResponse(status_code=400, content=error_body(str(bad), bad.param, bad.code))
        cam = getattr(app.state, "cam", None)
        if cam is not None:
            ns = request.headers.get("x-cam-namespace") or "default"
            last_user = payload if isinstance(payload, str) else next(
                (str(m.get("content") or "") for m in reversed(payload) if m.get("role") == "user"), "")
            cam_auto_write(cam, last_user, req.cam_write, ns)
            payload = cam_auto_read(cam, payload, req.cam_read, ns)
        kwargs = dict(req.chat_template_kwargs or {})
        if req.enable_thinking is not None:
            kwargs.setdefault("enable_thinking", req.enable_thinking)
        await state.send_one(TokenizeMsg(uid, payload, sp, kwargs or None, req.tools, images=images or None))
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        model = req.model or args.model_name
        obj = "chat.completion" if chat else "text_completion"
        use_reasoning = chat and reasoning is not None and req.enable_thinking is not False
        want_tools = chat and bool(req.tools) and req.tool_choice != "none"

        if req.stream:
            include_usage = bool((req.stream_options or {}).get("include_usage"))

            async def gen():
                rstate = ReasoningStreamState(reasoning, reasoning.starts_open) if use_reasoning else None
                tstate = ToolCallStreamState(req.tools, resolve_tool_format(None, chat_template)) if want_tools else None
                n_calls = 0
                n_tok = prompt_tok = cached = 0
                finish = None
                if chat:
                    yield _sse({"id": rid, "object": obj + ".chunk", "created": created, "model": model,
                                "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""},
                                             "finish_reason": None}]})
                async for reply in state.replies(uid):
                    if reply.error:
                        yield _sse({"error": {"message": reply.error, "type": "invalid_request_error"}})
                        finish = "error"
                        break
                    n_tok += len(reply.token_ids)
                    prompt_tok, cached = reply.prompt_tokens, reply.cached_tokens
                    text = reply.incremental_output
                    r_delta, c_delta = ("", text)
                    if rstate is not None:
                        r_delta, c_delta = rstate.feed(text)
                        if reply.finished:
                            r2, c2 = rstate.flush()
                            r_delta, c_delta = r_delta + r2, c_delta + c2
                    call_deltas: List[Dict[str, Any]] = []
                    if tstate is not None:
                        c_delta, call_deltas = tstate.push(c_delta)
                    delta: Dict[str, Any] = {}
                    if r_delta:
                        delta["reasoning_content"] = r_delta
                    if c_delta:
                        delta["content" if chat else "text"] = c_delta
                    if reply.logprobs:
                        delta_lp = {"content": reply.logprobs}
                    else:
                        delta_lp = None
                    if call_deltas:
                        # a call's name goes out as soon as it is complete, its arguments as they grow
                        delta["tool_calls"] = call_deltas
                        n_calls += sum(1 for c in call_deltas if "id" in c)
                    if delta:
                        choice = ({"index": 0, "delta": delta, "finish_reason": None} if chat
                                  else {"index": 0, "text": c_delta, "finish_reason": None})
                        if delta_lp:
                            choice["logprobs"] = delta_lp
                        yield _sse({"id": rid, "object": obj + (".chunk" if chat else ""), "created": created,
                                    "model": model, "choices": [choice]})
                    if reply.finished:
                        finish = reply.finish_reason or "stop"
                calls: List[Dict[str, Any]] = []
                if tstate is not None:
                    rest, calls = tstate.flush()
                    if rest:
                        yield _sse({"id": rid, "object": obj + ".chunk", "created": created, "model": model,
                                    "choices": [{"index": 0, "delta": {"content": rest}, "finish_reason": None}]})
                    if calls:
                        yield _sse({"id": rid, "object": obj + ".chunk", "created": created, "model": model,
                                    "choices": [{"index": 0, "delta": {"tool_calls": calls}, "finish_reason": None}]})
                    n_calls += sum(1 for c in calls if "id" in c)
                if n_calls and finish in (None, "stop"):
                    finish = "tool_calls"
                final = ({"index": 0, "delta": {}, "finish_reason": finish or "stop"} if chat
                         else {"index": 0, "text": "", "finish_reason": finish or "stop"})
                yield _sse({"id": rid, "object": obj + (".chunk" if chat else ""), "created": created, "model": model,
                            "choices": [final]})
                if include_usage:
                    yield _sse({"id": rid, "object": obj + (".chunk" if chat else ""), "created": created,
                                "model": model, "choices": [], "usage": _usage(prompt_tok, n_tok, cached)})
                yield _sse("[DONE]")

            return StreamingResponse(stream_with_cancellation(request, gen(), lambda: state.abort_user(uid)),
                                     media_type="text/event-stream")

        # ---- non-streaming
        text_parts: List[str] = []
        lp_records: List[Dict[str, Any]] = []
        n_tok = prompt_tok = cached = 0
        finish = "stop"
        try:
            async for reply in state.replies(uid):
                if await request.is_disconnected():
                    await state.abort_user(uid)
                    raise HTTPException(status_code=499, detail="client disconnected")
                if reply.error:
                    raise HTTPException(status_code=400, detail=reply.error)
                text_parts.append(reply.incremental_output)
                n_tok += len(reply.token_ids)
                prompt_tok, cached = reply.prompt_tokens, reply.cached_tokens
                if reply.logprobs:
                    lp_records.extend(reply.logprobs)
                if reply.finished:
                    finish = reply.finish_reason or "stop"
        except asyncio.CancelledError:
            await state.abort_user(uid)
            raise
        text = "".join(text_parts)
        if chat:
            reasoning_text = None
            if use_reasoning:
                reasoning_text, text = reasoning.split(text)
            calls: List[Dict[str, Any]] = []
            if want_tools:
                text, calls = parse_tool_calls(text, req.tools, resolve_tool_format(None, chat_template))
            message: Dict[str, Any] = {"role": "assistant", "content": text if (text or not calls) else None}
            if reasoning_text:
                message["reasoning_content"] = reasoning_text
            if calls:
                message["tool_calls"] = calls
                if finish == "stop":
                    finish = "tool_calls"
            choice: Dict[str, Any] = {"index": 0, "message": message, "finish_reason": finish}
        else:
            choice = {"index": 0, "text": text, "finish_reason": finish}
        if lp_records:
            choice["logprobs"] = {"content": lp_records}
        return JSONResponse({"id": rid, "object": obj, "created": created, "model": model, "choices": [choice],
                             "usage": _usage(prompt_tok, n_tok, cached)})

    if os.environ.get("MSGL_CAM", os.environ.get("MINISGL_CAM", "0")) == "1":
        # editable associative memory: /cam/* edit plane; /cam/ask answers through the served model
        from ..cam import CamMemory
        from .cam_api import make_cam_router

        cam_memory = CamMemory(os.environ.get("MSGL_CAM_PATH") or None,
                               int(os.environ.get("MSGL_CAM_MAX_NAMESPACES", "0") or 0))
        app.state.cam = cam_memory

        async def _cam_generate(prompt: str, max_tokens: int) -> str:
            state.ensure_listener()
            uid = state.new_user()
            await state.send_one(TokenizeMsg(uid, prompt, SamplingParams(temperature=0.0, max_tokens=max_tokens)))
            parts = []
            async for reply in state.replies(uid):
                if reply.error:
                    raise HTTPException(status_code=500, detail=reply.error)
                if reply.incremental_output:
                    parts.append(reply.incremental_output)
            return "".join(parts)

        app.include_router(make_cam_router(cam_memory, _cam_generate if state.send_queue is not None else None))

    def _rsa_params(req: OpenAICompletionRequest):
        """Recursive self-aggregation applies when the request asks for it (``rsa``), or, with the
        server's effort ladder enabled, when ``reasoning_effort`` maps to a ladder rung
        (python/minisgl/server/api_server.py:1204)."""
        from dataclasses import fields, replace

        from ..rsa import RSAParams

        base = getattr(args, "rsa", None) or RSAParams()
        if req.rsa:
            if isinstance(req.rsa, dict):
                allowed = {f.name for f in fields(RSAParams)}
                bad = sorted(set(req.rsa) - allowed)
                if bad:
                    raise HTTPException(status_code=400, detail=f"unknown rsa fields: {bad}")
                return replace(base, **req.rsa)
            return base
        if getattr(args, "rsa_effort_ladder", False) and req.reasoning_effort:
            return RSAParams.from_effort(req.reasoning_effort)
        return None

    async def _run_rsa(req: OpenAICompletionRequest, request: Request, params):
        from ..rsa import run_rsa

        if req.messages is None:
            raise HTTPException(status_code=400, detail="`messages` is required")
        if req.tools:
            raise HTTPException(status_code=400, detail="rsa does not combine with tools")
        state.ensure_listener()
        usage = {"prompt_tokens": 0, "completion_tokens": 0}

        async def generate(msgs, max_tokens, temperature, top_p) -> str:
            uid = state.new_user()
            sp = SamplingParams(temperature=float(temperature), top_p=float(top_p), max_tokens=int(max_tokens),
                                ignore_eos=False)
            await state.send_one(TokenizeMsg(uid, msgs, sp, dict(req.chat_template_kwargs or {}) or None, None))
            parts = []
            try:
                async for reply in state.replies(uid):
                    if reply.error:
                        raise RuntimeError(reply.error)
                    if reply.incremental_output:
                        parts.append(reply.incremental_output)
                    usage["completion_tokens"] += len(reply.token_ids)
                    if getattr(reply, "prompt_tokens", 0):
                        usage["prompt_tokens"] = max(usage["prompt_tokens"], int(reply.prompt_tokens))
            except asyncio.CancelledError:
                await state.abort_user(uid)
                raise
            text = "".join(parts)
            if reasoning is not None:   # candidates are aggregated on their answers, not on their thoughts
                text = reasoning.split(text)[1] if hasattr(reasoning, "split") else text
            return text

        messages = [m.model_dump(exclude_none=True) for m in req.messages]
        result = await run_rsa(messages, params, generate)
        rid = "chatcmpl-" + uuid.uuid4().hex[:24]
        model = req.model or args.model_name
        created = int(time.time())
        usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
        meta = {"rounds": result["rounds"], "calls": result["calls"], "n": params.n, "k": params.k, "t": params.t}
        if req.stream:
            async def gen():
                yield _sse({"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                            "choices": [{"index": 0, "delta": {"role": "assistant", "content": result["answer"]},
                                         "finish_reason": None}]})
                yield _sse({"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                            "choices": [{"index": 0, "delta": {}, "finish_reason": "stop"}], "usage": usage,
                            "rsa": meta})
                yield _sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")
        return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model,
                             "choices": [{"index": 0, "message": {"role": "assistant", "content": result["answer"]},
                                          "finish_reason": "stop"}], "usage": usage, "rsa": meta})

    @app.post("/v1/chat/completions")
    async def v1_chat_completions(req: OpenAICompletionRequest, request: Request):
        bad = reject_unclosed_tool_call(req.messages, resolve_tool_format(tokenizer, chat_template) if (
            tokenizer is not None or chat_template) else None)
        if bad is not None:
            return JSONResponse(status_code=400, content=error_body(str(bad), bad.param, bad.code))
        params = _rsa_params(req)
        if params is not None:
            return await _run_rsa(req, request, params)
        return await _run(req, request, chat=True)

    @app.post("/v1/completions")
    async def v1_completions(req: OpenAICompletionRequest, request: Request):
        # the raw-prompt lane: chat-only fields are errors, not silently dropped
        for cond, msg, param in (
                (req.messages is not None and req.prompt is None,
                 "`messages` is not accepted by /v1/completions: this endpoint continues a raw `prompt`", "messages"),
                (bool(req.tools), "`tools` are not supported by /v1/completions: tool specs are rendered by the chat template",
                 "tools"),
                (req.rsa not in (None, False), "`rsa` requires `messages` (chat format), not a raw `prompt`", "rsa")):
            if cond:
                return JSONResponse(status_code=400, content=error_body(msg, param, "unsupported_parameter"))
        return await _run(req, request, chat=False)

    return app


def run_api_server(args: ServerArgs, start_backend=None) -> None:
    """Create the ZMQ links, start the backend processes and serve with uvicorn."""
    import uvicorn

    from ..utils.mp import ZmqAsyncPullQueue, ZmqAsyncPushQueue
    from ..tokenizer.simple import load_tokenizer

    manager = FrontendManager(
        args, send_queue=ZmqAsyncPushQueue(args.zmq_tokenizer_addr, create=False),
        recv_queue=ZmqAsyncPullQueue(args.zmq_frontend_addr, create=True))
    template = args.chat_template
    tokenizer = None
    try:
        tokenizer = load_tokenizer(args.model_path)
    except Exception:
        tokenizer = None
    if template is None:
        template = getattr(tokenizer, "chat_template", None)
    defaults = set_sampling_defaults(args.model_path)
    if defaults:
        logger.info("sampling defaults from generation_config.json: %s", defaults)
    if start_backend is not None:
        start_backend()
    app = create_app(args, manager, template if isinstance(template, str) else None,
                     tokenizer if hasattr(tokenizer, "apply_chat_template") else None)
    uvicorn.run(app, host=args.host, port=args.port, log_level="warning")
