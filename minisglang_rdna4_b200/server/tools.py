"""Tool calling: which wire format a checkpoint speaks, grammars that constrain a call to that
format, parsers for generated calls (whole text and streaming).

Reference behaviour: python/minisgl/server/api_server.py:461-733 (grammar synthesis and format
derivation), :2149-2553 (parsers, type coercion, name policy), :2585-2936 (streaming state).

Formats (``ToolFormat``):

=============  ==========================================================================
``json``       ``<tool_call>{"name": …, "arguments": {…}}</tool_call>`` (Hermes / Qwen2.5 / Qwen3)
``qwen_xml``   ``<tool_call>\\n<function=NAME>\\n<parameter=P>\\nVALUE\\n</parameter>\\n</function>\\n</tool_call>``
``zaya_xml``   the same interior inside ``<zyphra_tool_call>``; also the inline ``<function=NAME(a='x', b=1)>``
``atem``       ``<atem:function_calls><atem:invoke name="N"><atem:parameter name="P">V</atem:parameter>…``
``gemma``      ``<|tool_call>call:NAME{key:value,…}<tool_call|>`` with bare keys and ``<|"|>`` string quotes
``laguna``     ``<tool_call>NAME<arg_key>k</arg_key><arg_value>v</arg_value>…</tool_call>``
``mistral``    ``[TOOL_CALLS][{"name": …, "arguments": {…}}, …]``
``llama_json`` ``<|python_tag|>{"name": …, "parameters": {…}}``
``pythonic``   ``[fn(a=1, b="x"), other()]``
=============  ==========================================================================

The format is read off the chat template (a probe conversation with one tool call is rendered and
the wrapper it prints is recognised); ``MSGL_TOOL_FORMAT`` pins it. XML-like formats carry no type
information, so parameter values are typed from the request's tool schemas: a declared string stays
the verbatim text even when it looks like JSON.
"""
from __future__ import annotations

import ast
import json
import os
import re
import uuid
from dataclasses import dataclass
from typing import Any, Dict, FrozenSet, List, Optional, Tuple

from ..utils.logger import init_logger

logger = init_logger(__name__)


@dataclass(frozen=True)
class ToolFormat:
    name: str
    opener: str
    closer: str                      # "" = the call runs to the end of the turn
    marks: Tuple[str, ...]           # all of these in a rendered tool call identify the format


FORMATS: Dict[str, ToolFormat] = {f.name: f for f in (
    ToolFormat("gemma", "<|tool_call>", "<tool_call|>", ("<|tool_call>call:",)),
    ToolFormat("atem", "<atem:function_calls>", "</atem:function_calls>", ("<atem:invoke",)),
    ToolFormat("zaya_xml", "<zyphra_tool_call>", "</zyphra_tool_call>", ("<zyphra_tool_call>",)),
    ToolFormat("qwen_xml", "<tool_call>", "</tool_call>", ("<tool_call>", "<function=")),
    ToolFormat("laguna", "<tool_call>", "</tool_call>", ("<tool_call>", "<arg_key>")),
    ToolFormat("mistral", "[TOOL_CALLS]", "", ("[TOOL_CALLS]",)),
    ToolFormat("llama_json", "<|python_tag|>", "", ("<|python_tag|>",)),
    ToolFormat("json", "<tool_call>", "</tool_call>", ("<tool_call>",)),
    ToolFormat("pythonic", "[", "]", ()),
)}
# order in which a rendered probe is matched: the more specific wrapper wins
_DERIVE_ORDER = ("gemma", "atem", "zaya_xml", "qwen_xml", "laguna", "mistral", "llama_json", "json")

TOOL_PROBE_MESSAGES = [
    {"role": "user", "content": "hi"},
    {"role": "assistant", "content": "", "tool_calls": [
        {"id": "c1", "type": "function", "function": {"name": "f", "arguments": {"k": "v"}}}]},
]
_TOOL_PROBE_TOOLS = [{"type": "function", "function": {
    "name": "f", "description": "d", "parameters": {"type": "object", "properties": {"k": {"type": "string"}}}}}]


def derive_tool_format(tokenizer=None, chat_template: Optional[str] = None) -> Optional[str]:
    """The checkpoint's own tool-call format. The template is the fact: with a tokenizer, a probe
    tool call is rendered through it and the wrapper read back; with only the template source, the
    wrapper literals are looked for in the text. ``None`` = nothing recognised (callers use ``json``)."""
    rendered = None
    if tokenizer is not None and hasattr(tokenizer, "apply_chat_template"):
        for kwargs in ({"tools": _TOOL_PROBE_TOOLS}, {}):
            try:
                rendered = tokenizer.apply_chat_template(TOOL_PROBE_MESSAGES, tokenize=False,
                                                         add_generation_prompt=False, **kwargs)
                break
            except Exception as exc:          # a template that rejects the probe says nothing
                logger.debug("tool-format probe failed: %s", exc)
    text = rendered if rendered is not None else (chat_template or "")
    if not text:
        return None
    for name in _DERIVE_ORDER:
        fmt = FORMATS[name]
        if all(m in text for m in fmt.marks):
            if name == "json" and rendered is None and "tool_call" not in text:
                continue
            return name
    return None


_RESOLVED: Dict[int, str] = {}


def resolve_tool_format(tokenizer=None, chat_template: Optional[str] = None) -> str:
    """``MSGL_TOOL_FORMAT`` unless it is unset or ``auto``; else the derived format; else ``json``."""
    pinned = os.environ.get("MSGL_TOOL_FORMAT", os.environ.get("MINISGL_TOOL_FORMAT", "auto")).strip()
    if pinned and pinned != "auto":
        if pinned not in FORMATS:
            raise ValueError(f"MSGL_TOOL_FORMAT={pinned!r}: known formats are {sorted(FORMATS)}")
        return pinned
    key = hash((id(tokenizer), chat_template))
    if key not in _RESOLVED:
        _RESOLVED[key] = derive_tool_format(tokenizer, chat_template) or "json"
        logger.info("tool-call format: %s", _RESOLVED[key])
    return _RESOLVED[key]


def tool_openers_closers(template: Optional[str], fmt: Optional[str] = None) -> Tuple[List[str], List[str]]:
    """Opener / closer strings the scheduler's tool gate follows for this checkpoint."""
    f = FORMATS[fmt or resolve_tool_format(None, template)]
    if f.name == "pythonic":
        return [], []
    return [f.opener], [f.closer] if f.closer else []


# ------------------------------------------------------------------------------------------ schemas
def _functions(tools: Optional[List[Dict[str, Any]]], forced: Optional[str] = None) -> List[Dict[str, Any]]:
    out = []
    for t in tools or ():
        fn = (t or {}).get("function") or (t if isinstance(t, dict) and "name" in t else None)
        if not fn or not fn.get("name") or (forced and fn["name"] != forced):
            continue
        out.append(fn)
    return out


def tool_param_types(tools) -> Dict[str, Dict[str, Optional[str]]]:
    """``{tool: {param: declared JSON type}}`` from the request's tool specs."""
    out: Dict[str, Dict[str, Optional[str]]] = {}
    for fn in _functions(tools):
        props = (fn.get("parameters") or {}).get("properties") or {}
        if isinstance(props, dict):
            out[fn["name"]] = {k: (v or {}).get("type") for k, v in props.items() if isinstance(v, dict)}
    return out


_BARE = {"true": True, "false": False, "null": None}


def coerce(val: str, expected: Optional[str] = None):
    """Raw parameter text of an untyped format -> the type the tool's schema declares. A declared
    string is returned verbatim. With no declaration only the unambiguous cases are converted
    (objects, arrays, true / false / null); a bare number or a quoted string stays text."""
    if expected == "string":
        return val
    if expected in ("integer", "number", "boolean", "array", "object"):
        try:
            return json.loads(val)
        except (json.JSONDecodeError, ValueError):
            return val
    s = val.strip()
    if s in _BARE:
        return _BARE[s]
    if s[:1] in ("{", "["):
        try:
            return json.loads(s)
        except (json.JSONDecodeError, ValueError):
            return val
    return val


def _rehome_refs(node, ns: str):
    """Rewrite local ``$ref`` targets (``#/$defs/X``, ``#/definitions/X``) into the namespace ``ns``."""
    if isinstance(node, dict):
        out = {}
        for k, v in node.items():
            if k == "$ref" and isinstance(v, str) and (v.startswith("#/$defs/") or v.startswith("#/definitions/")):
                out[k] = "#/$defs/" + ns + "__" + v.split("/", 2)[2]
            elif k in ("$defs", "definitions"):
                continue
            else:
                out[k] = _rehome_refs(v, ns)
        return out
    if isinstance(node, list):
        return [_rehome_refs(v, ns) for v in node]
    return node


def _hoist_defs(params: Dict[str, Any], ns: str, defs_out: Dict[str, Any]) -> Dict[str, Any]:
    """A tool's parameter schema may carry its own ``$defs``; several tools in one ``anyOf`` would
    collide, so each tool's definitions move to the root under a per-tool prefix."""
    for key in ("$defs", "definitions"):
        for name, sub in (params.get(key) or {}).items():
            defs_out[f"{ns}__{name}"] = _rehome_refs(sub, ns)
    return _rehome_refs(params, ns)


def _ebnf_lit(s: str) -> str:
    return '"' + s.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n") + '"'


def _names_and_params(fns) -> Tuple[str, str]:
    names = " | ".join(_ebnf_lit(f["name"]) for f in fns)
    params = sorted({p for f in fns for p in ((f.get("parameters") or {}).get("properties") or {})})
    return names, (" | ".join(_ebnf_lit(p) for p in params) if params else _ebnf_lit("_"))


def _xml_grammar(fns, opener: str, closer: str) -> str:
    names, params = _names_and_params(fns)
    return "\n".join([
        "root ::= " + _ebnf_lit(opener + "\n<function=") + " fname " + _ebnf_lit(">\n") + " param* "
        + _ebnf_lit("</function>\n" + closer),
        f"fname ::= {names}",
        'param ::= "<parameter=" pname ">\\n" pval "\\n</parameter>\\n"',
        f"pname ::= {params}",
        "pval ::= [^<]*",
    ])


def _atem_grammar(fns) -> str:
    names, params = _names_and_params(fns)
    return "\n".join([
        'root ::= "<atem:function_calls>\\n<atem:invoke name=\\"" fname "\\">\\n" param* '
        '"</atem:invoke>\\n</atem:function_calls>"',
        f"fname ::= {names}",
        'param ::= "<atem:parameter name=\\"" pname "\\">" pval "</atem:parameter>\\n"',
        f"pname ::= {params}",
        "pval ::= [^<]*",
    ])


def _gemma_grammar(fns) -> str:
    names, keys = _names_and_params(fns)
    q = _ebnf_lit('<|"|>')
    return "\n".join([
        'root ::= "<|tool_call>call:" fname "{" args "}<tool_call|>"',
        f"fname ::= {names}",
        'args ::= (arg ("," arg)*)?',
        'arg ::= key ":" value',
        f"key ::= {keys}",
        "value ::= str | bool | num | arr | obj",
        f"str ::= {q} schar* {q}",
        'schar ::= [^<] | "<" [^|]',          # anything but the two characters that start the closing quote
        'bool ::= "true" | "false"',
        'num ::= "-"? [0-9]+ ("." [0-9]+)?',
        'arr ::= "[" (value ("," value)*)? "]"',
        'obj ::= "{" (okv ("," okv)*)? "}"',
        'okv ::= ident ":" value',
        "ident ::= [a-zA-Z_] [a-zA-Z0-9_]*",
    ])


def _laguna_grammar(fns) -> str:
    names, params = _names_and_params(fns)
    return "\n".join([
        'root ::= "<tool_call>" fname pair* "</tool_call>"',
        f"fname ::= {names}",
        'pair ::= "<arg_key>" pname "</arg_key><arg_value>" pval "</arg_value>"',
        f"pname ::= {params}",
        "pval ::= [^<]*",
    ])


def grammar_from_tools(tools: List[Dict[str, Any]], tool_choice: Any, fmt: str = "json") -> Optional[str]:
    """Grammar spec (for ``engine.grammar``) of a *forced* call: ``tool_choice`` "required" allows any
    offered function, a named choice pins one; "auto" / "none" / absent return None (auto must stay
    free not to call). JSON-bodied formats give a JSON schema (``{"name": const, "arguments": schema}``
    per tool, ``$defs`` hoisted per tool); the native XML-like formats give an ``ebnf:`` grammar that
    pins function and parameter names and leaves values permissive."""
    if not tools or tool_choice in (None, "auto", "none"):
        return None
    forced = None
    if isinstance(tool_choice, dict):
        forced = (tool_choice.get("function") or {}).get("name") or tool_choice.get("name")
    elif tool_choice != "required":
        return None
    fns = _functions(tools, forced)
    if not fns:
        if forced:
            raise ValueError(f"tool_choice names an unknown function {forced!r}")
        return None
    if fmt in ("qwen_xml", "zaya_xml"):
        return "ebnf:" + _xml_grammar(fns, FORMATS[fmt].opener, FORMATS[fmt].closer)
    if fmt == "atem":
        return "ebnf:" + _atem_grammar(fns)
    if fmt == "gemma":
        return "ebnf:" + _gemma_grammar(fns)
    if fmt == "laguna":
        return "ebnf:" + _laguna_grammar(fns)
    variants, defs = [], {}
    arg_key = "parameters" if fmt == "llama_json" else "arguments"
    for i, f in enumerate(fns):
        params = _hoist_defs(dict(f.get("parameters") or {"type": "object"}), f"t{i}", defs)
        variants.append({"type": "object", "properties": {"name": {"const": f["name"]}, arg_key: params},
                         "required": ["name", arg_key], "additionalProperties": False})
    schema: Dict[str, Any] = variants[0] if len(variants) == 1 else {"anyOf": variants}
    if fmt == "mistral":
        schema = {"type": "array", "items": schema, "minItems": 1}
    if defs:
        schema = dict(schema, **{"$defs": defs})
    return json.dumps(schema)


def structural_tag_for_tools(tools: List[Dict[str, Any]], fmt: str = "json") -> Optional[str]:
    """``tool_choice: auto`` with a JSON-bodied format: free text until the opener appears, then the
    body is held to the offered tools' schemas (an xgrammar structural tag). Opt-in
    (``MSGL_TOOL_AUTO_CONSTRAIN=1``): a checkpoint trained on another body format would be masked
    off its own syntax."""
    if fmt != "json":
        return None
    f = FORMATS[fmt]
    structures = []
    for fn in _functions(tools):
        structures.append({"begin": f.opener + '\n{"name": "' + fn["name"] + '", "arguments": ',
                           "schema": fn.get("parameters") or {"type": "object"}, "end": "}\n" + f.closer})
    if not structures:
        return None
    return "structural_tag:" + json.dumps({"type": "structural_tag", "structures": structures, "triggers": [f.opener]})


# ------------------------------------------------------------------------------------------ parsers
_XML_FN = re.compile(r"<function=([^>(\s]+)\s*>(.*?)(?:</function>|\Z)", re.S)
_XML_PARAM = re.compile(r"<parameter=([^>]+)>\n?(.*?)\n?</parameter>", re.S)
_INLINE_FN = re.compile(r"<function=([A-Za-z_][\w.\-]*)\((.*)\)\s*>", re.S)
_ATEM_INVOKE = re.compile(r'<atem:invoke\s+name="([^"]+)"\s*>(.*?)</atem:invoke>', re.S)
_ATEM_PARAM = re.compile(r'<atem:parameter\s+name="([^"]+)"\s*>(.*?)</atem:parameter>', re.S)
_ARG_KV = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)
_TOOL_NAME = re.compile(r"[A-Za-z_][\w.\-]{0,63}")
_KV_FALLBACK = re.compile(r"""(\w+)\s*=\s*(?:'((?:[^'\\]|\\.)*)'|"((?:[^"\\]|\\.)*)"|([^,]+))""")
_GEMMA_CALL = re.compile(r"^call:([A-Za-z_][\w.\-]*)\s*(\{.*\})\s*$", re.S)


def parse_pycall_args(argstr: str) -> Dict[str, Any]:
    """Keyword arguments of an inline python-style call (``a='x', b=1, c=[1, 2]``). Clean literals go
    through ``ast``; otherwise a permissive ``key=value`` scan in which a quoted value is text and a
    bare value is a JSON literal if it parses as one."""
    argstr = argstr.strip()
    if not argstr:
        return {}
    try:
        call = ast.parse(f"_f({argstr})", mode="eval").body
        out = {kw.arg: ast.literal_eval(kw.value) for kw in getattr(call, "keywords", []) if kw.arg}
        if out:
            return out
    except Exception:
        pass
    out = {}
    for m in _KV_FALLBACK.finditer(argstr):
        single, double, bare = m.group(2), m.group(3), m.group(4)
        if single is not None or double is not None:
            out[m.group(1)] = single if single is not None else double
            continue
        raw = (bare or "").strip()
        try:
            out[m.group(1)] = json.loads(raw)
        except (json.JSONDecodeError, ValueError):
            out[m.group(1)] = raw
    return out


def gemma_args_to_json(text: str) -> str:
    """Gemma's argument object (bare keys, strings between ``<|"|>``) as JSON text, in one pass that
    tracks whether the cursor is inside a string."""
    out: List[str] = []
    i, n = 0, len(text)
    quote = '<|"|>'
    while i < n:
        if text.startswith(quote, i):
            j = text.find(quote, i + len(quote))
            if j == -1:
                j = n
            out.append(json.dumps(text[i + len(quote):j]))
            i = j + len(quote)
            continue
        m = re.match(r"[A-Za-z_][\w\-]*", text[i:])
        if m:
            word = m.group(0)
            k = i + len(word)
            while k < n and text[k] == " ":
                k += 1
            if k < n and text[k] == ":" and word not in _BARE:
                out.append(json.dumps(word))           # a bare key
            else:
                out.append(word)                       # true / false / null, or a bare word value
            i += len(word)
            continue
        out.append(text[i])
        i += 1
    return "".join(out)


def parse_gemma_call(inner: str) -> Optional[Tuple[str, Dict[str, Any]]]:
    m = _GEMMA_CALL.match(inner.strip())
    if not m:
        return None
    try:
        args = json.loads(gemma_args_to_json(m.group(2)))
    except (json.JSONDecodeError, ValueError):
        return None
    return (m.group(1), args) if isinstance(args, dict) else None


def parse_one_call(inner: str, param_types: Optional[Dict[str, Dict[str, Optional[str]]]] = None
                   ) -> Optional[Tuple[str, Dict[str, Any]]]:
    """One wrapper body -> ``(name, arguments)``, or None when it is not a call in any known form."""
    inner = inner.strip()
    pt = lambda fn, p: ((param_types or {}).get(fn) or {}).get(p)
    hit = parse_gemma_call(inner)               # before the bare-name form, whose head it would match
    if hit is not None:
        return hit
    if inner.startswith("{"):
        try:
            obj = json.loads(inner)
            name = obj.get("name") or (obj.get("function") or {}).get("name")
            if isinstance(name, str) and name:
                args = obj.get("arguments", obj.get("parameters", (obj.get("function") or {}).get("arguments", {})))
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except (json.JSONDecodeError, ValueError):
                        pass
                return name, args
        except (json.JSONDecodeError, ValueError, AttributeError):
            pass
    m = _ATEM_INVOKE.search(inner)
    if m and m.group(1).strip():
        fn = m.group(1).strip()
        return fn, {k.strip(): coerce(v, pt(fn, k.strip())) for k, v in _ATEM_PARAM.findall(m.group(2))}
    m = _INLINE_FN.search(inner)
    if m:
        return m.group(1).strip(), parse_pycall_args(m.group(2))
    m = _XML_FN.search(inner)
    if m:
        fn = m.group(1).strip()
        return fn, {k.strip(): coerce(v, pt(fn, k.strip())) for k, v in _XML_PARAM.findall(m.group(2))}
    if inner and not inner.startswith(("{", "<", "[")):
        name = inner.split("<", 1)[0].strip()
        # the head must look like a function name: an unparsed body is visible, a wrong call is dispatched
        if name and _TOOL_NAME.fullmatch(name):
            return name, {k.strip(): coerce(v.strip(), pt(name, k.strip())) for k, v in _ARG_KV.findall(inner)}
    return None


def parse_pythonic(text: str) -> List[Tuple[str, Dict[str, Any]]]:
    """``[fn(a=1), other(b="x")]`` -> calls; ``[]`` when the text is not such a list."""
    s = text.strip()
    if not (s.startswith("[") and s.endswith("]")):
        return []
    try:
        node = ast.parse(s, mode="eval").body
    except SyntaxError:
        return []
    if not isinstance(node, ast.List) or not node.elts:
        return []
    calls = []
    for el in node.elts:
        if not isinstance(el, ast.Call) or el.args:
            return []
        fn = el.func
        name = fn.id if isinstance(fn, ast.Name) else (ast.unparse(fn) if isinstance(fn, ast.Attribute) else None)
        if not name:
            return []
        try:
            calls.append((name, {kw.arg: ast.literal_eval(kw.value) for kw in el.keywords if kw.arg}))
        except (ValueError, SyntaxError):
            return []
    return calls


UNKNOWN_TOOL_SEEN: Dict[str, int] = {}


def known_tool_names(tools) -> Optional[FrozenSet[str]]:
    names = frozenset(f["name"] for f in _functions(tools))
    return names or None


def tool_name_allowed(name: str, allowed: Optional[FrozenSet[str]]) -> bool:
    """A call to a function that was not offered is forwarded (the client answers with a tool error
    and the model corrects itself next turn) unless ``MSGL_DROP_UNKNOWN_TOOLS=1``; counted either way."""
    if allowed is None or name in allowed:
        return True
    UNKNOWN_TOOL_SEEN[name] = UNKNOWN_TOOL_SEEN.get(name, 0) + 1
    drop = os.environ.get("MSGL_DROP_UNKNOWN_TOOLS", os.environ.get("MINISGL_DROP_UNKNOWN_TOOLS")) == "1"
    if UNKNOWN_TOOL_SEEN[name] == 1:
        logger.warning("%s tool call to %r, which the request did not offer", "dropped" if drop else "forwarding", name)
    return not drop


def make_call(name: str, args: Any) -> Dict[str, Any]:
    if not isinstance(args, str):
        args = json.dumps(args, ensure_ascii=False)
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function", "function": {"name": name, "arguments": args}}


def _json_values(blob: str) -> List[Any]:
    blob = blob.strip()
    try:
        val = json.loads(blob)
        return val if isinstance(val, list) else [val]
    except (json.JSONDecodeError, ValueError):
        pass
    out, dec, i = [], json.JSONDecoder(), 0
    while i < len(blob):
        j = blob.find("{", i)
        if j == -1:
            break
        try:
            val, end = dec.raw_decode(blob, j)
            out.append(val)
            i = end
        except json.JSONDecodeError:
            i = j + 1
    return out


_WRAPPERS: Tuple[Tuple[str, str], ...] = (
    ("<|tool_call>", "<tool_call|>"), ("<atem:function_calls>", "</atem:function_calls>"),
    ("<zyphra_tool_call>", "</zyphra_tool_call>"), ("<tool_call>", "</tool_call>"),
    ("<|tool_call|>", "<|/tool_call|>"), ("[TOOL_CALLS]", ""), ("<|python_tag|>", ""),
)


def parse_tool_calls(text: str, tools: Optional[List[Dict[str, Any]]] = None, fmt: Optional[str] = None
                     ) -> Tuple[str, List[Dict[str, Any]]]:
    """Split a completion into plain content and OpenAI-style tool calls. Every known wrapper is
    looked for (a model does not always answer in the format its template renders); a block that
    does not parse is left in the content."""
    allowed = known_tool_names(tools)
    types = tool_param_types(tools)
    calls: List[Dict[str, Any]] = []
    content = text

    def add(name: str, args: Any) -> None:
        if tool_name_allowed(name, allowed):
            calls.append(make_call(name, args))

    for opener, closer in _WRAPPERS:
        if opener not in content:
            continue
        if closer:
            pat = re.compile(re.escape(opener) + r"(.*?)(?:" + re.escape(closer) + r"|\Z)", re.S)
            kept: List[str] = []
            pos = 0
            for m in pat.finditer(content):
                body = m.group(1)
                parsed: List[Tuple[str, Any]] = []
                if opener == "<atem:function_calls>":      # one block may hold several invokes
                    for inv in _ATEM_INVOKE.finditer(body):
                        fn = inv.group(1).strip()
                        parsed.append((fn, {k.strip(): coerce(v, (types.get(fn) or {}).get(k.strip()))
                                            for k, v in _ATEM_PARAM.findall(inv.group(2))}))
                else:
                    one = parse_one_call(body, types)
                    if one is not None:
                        parsed.append(one)
                    elif body.strip().startswith("["):
                        for v in _json_values(body):
                            if isinstance(v, dict) and v.get("name"):
                                parsed.append((v["name"], v.get("arguments", v.get("parameters", {}))))
                kept.append(content[pos:m.start()])
                if parsed:
                    for name, args in parsed:
                        add(name, args)
                else:
                    kept.append(m.group(0))                # malformed: stays visible
                pos = m.end()
            kept.append(content[pos:])
            content = "".join(kept)
        else:
            head, _, tail = content.partition(opener)
            found = False
            for v in _json_values(tail):
                if isinstance(v, dict) and (v.get("name") or (v.get("function") or {}).get("name")):
                    name = v.get("name") or v["function"]["name"]
                    add(name, v.get("arguments", v.get("parameters", (v.get("function") or {}).get("arguments", {}))))
                    found = True
            if found:
                content = head
    if not calls and (fmt == "pythonic" or (fmt is None and tools)):
        py = parse_pythonic(content)
        if py and (allowed is None or fmt == "pythonic" or all(n in allowed for n, _ in py)):
            for name, args in py:
                add(name, args)
            if calls:
                content = ""
    if not calls and fmt == "llama_json" and content.strip().startswith("{"):
        for v in _json_values(content):
            if isinstance(v, dict) and v.get("name") and ("parameters" in v or "arguments" in v):
                add(v["name"], v.get("parameters", v.get("arguments", {})))
        if calls:
            content = ""
    return (content.strip() if calls else text), calls


# ------------------------------------------------------------------------------------------ streaming
class _JsonArgStreamer:
    """Follows a JSON call body ``{"name": "...", "arguments": {...}}`` as it grows: reports the
    name once it is complete and the argument text in increments, so a client sees the arguments
    arrive instead of one burst at the closer."""

    _NAME = re.compile(r'"name"\s*:\s*"((?:[^"\\]|\\.)*)"')
    _ARGS = re.compile(r'"(?:arguments|parameters)"\s*:\s*')

    def __init__(self) -> None:
        self.name: Optional[str] = None
        self.arg_start = -1
        self.sent = 0

    def scan(self, body: str) -> Tuple[Optional[str], str, bool]:
        """Returns ``(name once, new argument text, arguments complete)`` for the body so far."""
        new_name = None
        if self.name is None:
            m = self._NAME.search(body)
            if m:
                try:
                    self.name = new_name = json.loads('"' + m.group(1) + '"')
                except ValueError:
                    self.name = new_name = m.group(1)
        if self.name is None:
            return None, "", False
        if self.arg_start < 0:
            m = self._ARGS.search(body)
            if not m:
                return new_name, "", False
            self.arg_start = m.end()
        # the end of the argument value: bracket matching outside strings
        depth, in_str, esc, end = 0, False, False, -1
        for i in range(self.arg_start, len(body)):
            ch = body[i]
            if in_str:
                if esc:
                    esc = False
                elif ch == "\\":
                    esc = True
                elif ch == '"':
                    in_str = False
                    if depth == 0:
                        end = i + 1
                        break
                continue
            if ch == '"':
                in_str = True
            elif ch in "{[":
                depth += 1
            elif ch in "}]":
                depth -= 1
                if depth == 0:
                    end = i + 1
                    break
                if depth < 0:
                    end = i
                    break
        stop = end if end >= 0 else len(body)
        delta = body[self.arg_start + self.sent:stop]
        self.sent += len(delta)
        return new_name, delta, end >= 0


class ToolCallStreamState:
    """Streaming split of content and tool calls. ``push(delta)`` returns ``(content, tool_call
    deltas)``: content is forwarded until an opener (or a prefix of one at the end of the text)
    appears; a JSON-bodied call streams its name and argument text as they arrive; other bodies are
    held until their closer and emitted whole. ``flush()`` handles what is left at the end of the
    turn (an unclosed block is parsed as far as it goes, else returned as content)."""

    def __init__(self, tools: Optional[List[Dict[str, Any]]] = None, fmt: Optional[str] = None) -> None:
        self.tools = tools
        self.fmt = fmt
        self.allowed = known_tool_names(tools)
        self.types = tool_param_types(tools)
        self.buf = ""                       # text not yet forwarded as content
        self.in_call: Optional[Tuple[str, str]] = None
        self.index = 0                      # next tool-call index
        self._js: Optional[_JsonArgStreamer] = None
        self._js_id: Optional[str] = None
        self._js_skip = False

    # -- helpers
    @property
    def held_chars(self) -> int:
        return len(self.buf)

    def _openers(self) -> List[Tuple[str, str]]:
        if self.fmt and self.fmt != "pythonic":
            f = FORMATS[self.fmt]
            first = [(f.opener, f.closer)]
            return first + [w for w in _WRAPPERS if w[0] != f.opener]
        return list(_WRAPPERS)

    def _earliest(self, text: str) -> Tuple[int, Optional[Tuple[str, str]]]:
        best, which = -1, None
        for o, c in self._openers():
            p = text.find(o)
            if p != -1 and (best == -1 or p < best):
                best, which = p, (o, c)
        return best, which

    def _partial(self, text: str) -> int:
        hold = 0
        for o, _ in self._openers():
            for k in range(min(len(o) - 1, len(text)), 0, -1):
                if text.endswith(o[:k]):
                    hold = max(hold, k)
                    break
        return hold

    def _emit_whole(self, name: str, args: Any) -> List[Dict[str, Any]]:
        if not tool_name_allowed(name, self.allowed):
            return []
        call = make_call(name, args)
        call["index"] = self.index
        self.index += 1
        return [call]

    def _json_progress(self, body: str) -> List[Dict[str, Any]]:
        out: List[Dict[str, Any]] = []
        if self._js is None:
            self._js = _JsonArgStreamer()
        name, delta, _ = self._js.scan(body)
        if name is not None:
            self._js_skip = not tool_name_allowed(name, self.allowed)
            if not self._js_skip:
                self._js_id = "call_" + uuid.uuid4().hex[:24]
                out.append({"index": self.index, "id": self._js_id, "type": "function",
                            "function": {"name": name, "arguments": ""}})
        if delta and self._js.name is not None and not self._js_skip:
            out.append({"index": self.index, "function": {"arguments": delta}})
        return out

    def _close_json(self) -> None:
        if self._js is not None and self._js.name is not None and not self._js_skip:
            self.index += 1
        self._js, self._js_id, self._js_skip = None, None, False

    # -- API
    def push(self, delta: str) -> Tuple[str, List[Dict[str, Any]]]:
        self.buf += delta
        content_out: List[str] = []
        calls: List[Dict[str, Any]] = []
        while True:
            if self.in_call is None:
                pos, which = self._earliest(self.buf)
                if pos == -1:
                    hold = self._partial(self.buf)
                    cut = len(self.buf) - hold
                    content_out.append(self.buf[:cut])
                    self.buf = self.buf[cut:]
                    break
                content_out.append(self.buf[:pos])
                self.buf = self.buf[pos + len(which[0]):]
                self.in_call = which
                continue
            opener, closer = self.in_call
            end = self.buf.find(closer) if closer else -1
            body = self.buf if end == -1 else self.buf[:end]
            stripped = body.lstrip()
            if stripped.startswith("{") and closer:
                calls.extend(self._json_progress(stripped))
                if end == -1:
                    break
                if self._js is None or self._js.name is None:      # never became a call: give the text back
                    content_out.append(opener + body + closer)
                self._close_json()
            else:
                if end == -1:
                    break
                one = parse_one_call(body, self.types)
                if one is not None:
                    calls.extend(self._emit_whole(*one))
                else:
                    emitted = False
                    if opener == "<atem:function_calls>":
                        for inv in _ATEM_INVOKE.finditer(body):
                            fn = inv.group(1).strip()
                            calls.extend(self._emit_whole(fn, {k.strip(): coerce(v, (self.types.get(fn) or {}).get(k.strip()))
                                                               for k, v in _ATEM_PARAM.findall(inv.group(2))}))
                            emitted = True
                    if not emitted:
                        content_out.append(opener + body + closer)
            self.buf = self.buf[end + len(closer):]
            self.in_call = None
        return "".join(content_out), calls

    def flush(self) -> Tuple[str, List[Dict[str, Any]]]:
        """End of the turn: ``(remaining content, remaining tool-call deltas)``."""
        if self.in_call is None:
            rest, self.buf = self.buf, ""
            if self.index == 0 and rest.strip() and (self.fmt == "pythonic" or self.tools):
                text, calls = parse_tool_calls(rest, self.tools, self.fmt)
                if calls:
                    for c in calls:
                        c["index"] = self.index
                        self.index += 1
                    return "", calls
            return rest, []
        opener, closer = self.in_call
        body, self.buf, self.in_call = self.buf, "", None
        if self._js is not None and self._js.name is not None:
            calls = self._json_progress(body.lstrip())
            self._close_json()
            return "", calls
        self._close_json()
        _, calls = parse_tool_calls(opener + body, self.tools, self.fmt)
        if calls:
            for c in calls:
                c["index"] = self.index
                self.index += 1
            return "", calls
        return opener + body, []

    # compatibility with the earlier two-call interface
    def feed(self, delta: str) -> str:
        content, calls = self.push(delta)
        self._pending = getattr(self, "_pending", []) + calls
        return content

    def finish(self) -> Tuple[str, List[Dict[str, Any]]]:
        rest, calls = self.flush()
        return rest, getattr(self, "_pending", []) + calls
