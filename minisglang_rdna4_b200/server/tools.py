"""Tool calling: grammar synthesis for forced calls, parsing of generated calls (whole text
and streaming) for the common wire formats (python/minisgl/server/api_server.py:461-670
grammar synthesis, :2429 parsing, :2708 streaming state)."""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

# opener -> closer of the wrappers models emit around a JSON call
TOOL_WRAPPERS: Tuple[Tuple[str, str], ...] = (
    ("<tool_call>", "</tool_call>"),
    ("<|tool_call|>", "<|/tool_call|>"),
    ("[TOOL_CALLS]", ""),
    ("<|python_tag|>", ""),
)


def tool_openers_closers(template: Optional[str]) -> Tuple[List[str], List[str]]:
    """Wrappers that the chat template mentions (all known ones when it mentions none)."""
    found = [(o, c) for o, c in TOOL_WRAPPERS if template and o in template]
    pairs = found or [TOOL_WRAPPERS[0]]
    return [o for o, _ in pairs], [c for _, c in pairs if c]


def grammar_from_tools(tools: List[Dict[str, Any]], tool_choice: Any) -> Optional[str]:
    """JSON-schema grammar for a *required* call: ``tool_choice`` "required" allows any of the
    offered functions, a named choice pins one. Returns None when nothing is forced."""
    if not tools or tool_choice in (None, "auto", "none"):
        return None
    fns = [t.get("function", t) for t in tools]
    if isinstance(tool_choice, dict):
        name = (tool_choice.get("function") or {}).get("name") or tool_choice.get("name")
        fns = [f for f in fns if f.get("name") == name]
        if not fns:
            raise ValueError(f"tool_choice names an unknown function {name!r}")
    variants = []
    for f in fns:
        variants.append({
            "type": "object",
            "properties": {"name": {"const": f["name"]},
                           "arguments": f.get("parameters") or {"type": "object"}},
            "required": ["name", "arguments"], "additionalProperties": False,
        })
    schema = variants[0] if len(variants) == 1 else {"anyOf": variants}
    return json.dumps(schema)


def _make_call(obj: Dict[str, Any]) -> Optional[Dict[str, Any]]:
    name = obj.get("name") or (obj.get("function") or {}).get("name")
    if not isinstance(name, str):
        return None
    args = obj.get("arguments", obj.get("parameters", (obj.get("function") or {}).get("arguments", {})))
    if not isinstance(args, str):
        args = json.dumps(args, ensure_ascii=False)
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
            "function": {"name": name, "arguments": args}}


def _json_candidates(blob: str) -> List[Dict[str, Any]]:
    blob = blob.strip()
    out: List[Dict[str, Any]] = []
    try:
        val = json.loads(blob)
        vals = val if isinstance(val, list) else [val]
        return [v for v in vals if isinstance(v, dict)]
    except json.JSONDecodeError:
        pass
    dec = json.JSONDecoder()
    i = 0
    while i < len(blob):
        j = blob.find("{", i)
        if j == -1:
            break
        try:
            val, end = dec.raw_decode(blob, j)
            if isinstance(val, dict):
                out.append(val)
            i = end
        except json.JSONDecodeError:
            i = j + 1
    return out


def parse_tool_calls(text: str) -> Tuple[str, List[Dict[str, Any]]]:
    """Split generated text into plain content and OpenAI-style tool calls."""
    calls: List[Dict[str, Any]] = []
    content = text
    for opener, closer in TOOL_WRAPPERS:
        if opener not in content:
            continue
        if closer:
            pat = re.compile(re.escape(opener) + r"(.*?)(?:" + re.escape(closer) + r"|$)", re.S)
            for m in pat.finditer(content):
                for obj in _json_candidates(m.group(1)):
                    call = _make_call(obj)
                    if call:
                        calls.append(call)
            content = pat.sub("", content)
        else:
            head, _, tail = content.partition(opener)
            for obj in _json_candidates(tail):
                call = _make_call(obj)
                if call:
                    calls.append(call)
            content = head
    return content.strip() if calls else text, calls


@dataclass
class ToolCallStreamState:
    """Streaming: plain content is forwarded until an opener appears; everything after it is
    buffered and parsed when the stream ends (or the closer arrives)."""

    openers: List[str] = field(default_factory=lambda: [o for o, _ in TOOL_WRAPPERS])
    buf: str = ""
    in_call: bool = False
    emitted: int = 0

    def feed(self, delta: str) -> str:
        """Returns the content delta that is safe to forward."""
        self.buf += delta
        if self.in_call:
            return ""
        first = min((p for p in (self.buf.find(o) for o in self.openers) if p != -1), default=-1)
        if first != -1:
            out = self.buf[self.emitted:first]
            self.emitted = first
            self.in_call = True
            return out
        hold = 0
        for o in self.openers:
            for k in range(min(len(o) - 1, len(self.buf)), 0, -1):
                if self.buf.endswith(o[:k]):
                    hold = max(hold, k)
                    break
        end = len(self.buf) - hold
        out = self.buf[self.emitted:end] if end > self.emitted else ""
        self.emitted = max(self.emitted, end)
        return out

    def finish(self) -> Tuple[str, List[Dict[str, Any]]]:
        """Returns ``(remaining content, tool calls)``."""
        rest = self.buf[self.emitted:]
        if not self.in_call:
            return rest, []
        _, calls = parse_tool_calls(rest)
        return ("" if calls else rest), calls
