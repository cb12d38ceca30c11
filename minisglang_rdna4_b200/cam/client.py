"""Client for the memory plane of a running server (python/minisgl/cam/client.py:23-146).

Standard library only (``urllib``), so a script that talks to a server needs nothing installed beside this
file's package. ``transport`` replaces the HTTP call for tests or for an in-process application: a callable
``(method, path, headers, json_body) -> (status, parsed_json)``.
"""
from __future__ import annotations

import json
import urllib.error
import urllib.parse
import urllib.request
from typing import Any, Callable, Dict, List, Optional, Tuple


class CamError(RuntimeError):
    def __init__(self, status: int, detail: str) -> None:
        super().__init__(f"{status}: {detail}")
        self.status, self.detail = status, detail


Transport = Callable[[str, str, Dict[str, str], Optional[dict]], Tuple[int, Any]]


class CamClient:
    def __init__(self, base_url: str = "http://127.0.0.1:8000", token: Optional[str] = None,
                 namespace: Optional[str] = None, timeout: float = 30.0, transport: Optional[Transport] = None) -> None:
        self.base_url, self.token, self._ns, self.timeout = base_url.rstrip("/"), token, namespace, timeout
        self._transport = transport or self._http

    def namespace(self, ns: Optional[str]) -> "CamClient":
        """The same server and token, another namespace."""
        return CamClient(self.base_url, self.token, ns, self.timeout, self._transport if self._transport != self._http
                         else None)

    # ---- plumbing ----
    def _headers(self) -> Dict[str, str]:
        h = {"Content-Type": "application/json"}
        if self.token:
            h["Authorization"] = f"Bearer {self.token}"
        if self._ns:
            h["X-CAM-Namespace"] = self._ns
        return h

    def _http(self, method: str, path: str, headers: Dict[str, str], body: Optional[dict]) -> Tuple[int, Any]:
        data = json.dumps(body).encode() if body is not None else None
        req = urllib.request.Request(self.base_url + path, data=data, headers=headers, method=method)
        try:
            with urllib.request.urlopen(req, timeout=self.timeout) as resp:
                return resp.status, json.loads(resp.read().decode() or "null")
        except urllib.error.HTTPError as exc:
            raw = exc.read().decode()
            try:
                return exc.code, json.loads(raw)
            except ValueError:
                return exc.code, {"detail": raw}

    def _call(self, method: str, path: str, body: Optional[dict] = None) -> Any:
        status, payload = self._transport(method, path, self._headers(), body)
        if status >= 400:
            detail = payload.get("detail", payload) if isinstance(payload, dict) else payload
            raise CamError(status, str(detail))
        return payload

    # ---- operations ----
    def remember(self, subject: str, object: str, prompt: str = "") -> dict:
        return self._call("POST", "/cam/remember", {"subject": subject, "prompt": prompt, "object": object})

    def ask(self, prompt: str, subject: Optional[str] = None, max_tokens: int = 64) -> dict:
        return self._call("POST", "/cam/ask", {"prompt": prompt, "subject": subject, "max_tokens": max_tokens})

    def facts(self) -> List[dict]:
        return self._call("GET", "/cam/facts")

    def forget(self, subject: str) -> bool:
        return bool(self._call("DELETE", "/cam/facts/" + urllib.parse.quote(subject, safe=""))["deleted"])

    def undo(self) -> str:
        return self._call("POST", "/cam/undo")["undone"]

    def namespaces(self) -> List[str]:
        return self._call("GET", "/cam/namespaces")
