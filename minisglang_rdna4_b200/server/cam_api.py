"""``/cam/*`` edit plane of the associative memory (python/minisgl/server/cam_api.py:286-603):

    POST   /cam/remember          {subject, prompt, object}   -> {stored, replaced}
    POST   /cam/ask               {prompt, subject?, max_tokens?} -> {text, facts}
    GET    /cam/facts                                          -> [{subject, prompt, object}, ...]
    DELETE /cam/facts/{subject}                                -> {deleted}
    POST   /cam/undo                                           -> {undone}
    GET    /cam/namespaces                                     -> [namespace, ...]

Mounted only when ``MSGL_CAM=1``. The namespace comes from the ``X-CAM-Namespace`` header.
Authorisation: ``MSGL_CAM_TOKENS`` is JSON ``{token: "<ns>" | ["<ns>", ...] | "*"}``;
``MSGL_CAM_API_TOKEN`` is a single token for every namespace; with neither set the plane is open
(local use). A token may only touch its own namespaces (403 otherwise).
"""
from __future__ import annotations

import json
import os
from typing import Awaitable, Callable, Dict, List, Optional, Union

from fastapi import APIRouter, Depends, Header, HTTPException, Request
from pydantic import BaseModel

from ..cam import CamMemory

_ANY = "*"


class RememberBody(BaseModel):
    subject: str
    prompt: str = ""
    object: str


class AskBody(BaseModel):
    prompt: str
    subject: Optional[str] = None
    max_tokens: int = 64


def _token_table() -> Dict[str, Union[str, List[str]]]:
    table: Dict[str, Union[str, List[str]]] = {}
    single = os.environ.get("MSGL_CAM_API_TOKEN") or os.environ.get("MINISGL_CAM_API_TOKEN")
    if single:
        table[single] = _ANY
    raw = os.environ.get("MSGL_CAM_TOKENS") or os.environ.get("MINISGL_CAM_TOKENS")
    if raw:
        table.update(json.loads(raw))
    return table


def make_cam_router(memory: CamMemory,
                    generate: Optional[Callable[[str, int], Awaitable[str]]] = None) -> APIRouter:
    """``generate(prompt, max_tokens)`` runs the served model; without it ``/cam/ask`` returns the
    retrieved facts only."""
    tokens = _token_table()

    def principal(authorization: Optional[str] = Header(None)):
        if not tokens:
            return _ANY
        if not authorization or not authorization.startswith("Bearer "):
            raise HTTPException(status_code=401, detail="missing CAM API token")
        allowed = tokens.get(authorization[len("Bearer "):])
        if allowed is None:
            raise HTTPException(status_code=401, detail="invalid CAM API token")
        return allowed

    def namespace(request: Request, allowed=Depends(principal),
                  x_cam_namespace: Optional[str] = Header(None)) -> str:
        ns = x_cam_namespace or "default"
        if request.url.path.rstrip("/").endswith("/cam/namespaces"):
            return ns
        if allowed != _ANY and ns not in ([allowed] if isinstance(allowed, str) else list(allowed)):
            raise HTTPException(status_code=403, detail="token may not touch this namespace")
        return ns

    router = APIRouter(prefix="/cam", tags=["cam"])

    @router.post("/remember")
    async def remember(body: RememberBody, ns: str = Depends(namespace)):
        replaced = any(f.subject == body.subject.strip() for f in memory.facts(ns))
        try:
            memory.remember(body.subject, body.prompt, body.object, ns)
        except ValueError as exc:
            raise HTTPException(status_code=400, detail=str(exc))
        except PermissionError as exc:
            raise HTTPException(status_code=429, detail=str(exc))
        return {"stored": True, "replaced": replaced}

    @router.post("/ask")
    async def ask(body: AskBody, ns: str = Depends(namespace)):
        hits = memory.lookup(body.prompt if body.subject is None else body.subject + " " + body.prompt, ns)
        facts = [{"subject": f.subject, "object": f.object, "score": round(s, 4)} for s, f in hits]
        if generate is None:
            return {"text": hits[0][1].object if hits else "", "facts": facts}
        text = await generate(memory.augment(body.prompt, ns, body.subject), int(body.max_tokens))
        return {"text": text, "facts": facts}

    @router.get("/facts")
    async def facts(ns: str = Depends(namespace)):
        return [{"subject": f.subject, "prompt": f.prompt, "object": f.object} for f in memory.facts(ns)]

    @router.delete("/facts/{subject}")
    async def delete(subject: str, ns: str = Depends(namespace)):
        return {"deleted": memory.forget(subject, ns)}

    @router.post("/undo")
    async def undo(ns: str = Depends(namespace)):
        return {"undone": memory.undo(ns)}

    @router.get("/namespaces")
    async def namespaces(allowed=Depends(principal), _ns: str = Depends(namespace)):
        names = memory.namespaces()
        if allowed == _ANY:
            return names
        mine = [allowed] if isinstance(allowed, str) else list(allowed)
        return [n for n in names if n in mine]

    return router
