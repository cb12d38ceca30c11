"""Tool-call formats: derivation from the chat template, grammars for forced calls, parsers and
the streaming state (reference behaviour: python/minisgl/server/api_server.py:461-733, 2149-2936)."""
import json

import pytest

from minisglang_rdna4_b200.server import tools as T

TOOLS = [
    {"type": "function", "function": {"name": "run", "parameters": {"type": "object", "properties": {
        "command": {"type": "string"}, "timeout_s": {"type": "integer"}, "local": {"type": "boolean"}}}}},
    {"type": "function", "function": {"name": "web_search", "parameters": {"type": "object", "properties": {
        "query": {"type": "string"}, "limit": {"type": "integer"}}}}},
]


def _args(call):
    return json.loads(call["function"]["arguments"])


def test_format_is_read_off_the_template():
    assert T.derive_tool_format(None, "{{ '<tool_call>' }}{{ call | tojson }}{{ '</tool_call>' }}") == "json"
    assert T.derive_tool_format(None, "<tool_call>\n<function={{ name }}>\n<parameter={{ k }}>") == "qwen_xml"
    assert T.derive_tool_format(None, "<zyphra_tool_call><function=") == "zaya_xml"
    assert T.derive_tool_format(None, "'<|tool_call>call:' + name + '{'") == "gemma"
    assert T.derive_tool_format(None, '<atem:invoke name="') == "atem"
    assert T.derive_tool_format(None, "[TOOL_CALLS] [") == "mistral"
    assert T.derive_tool_format(None, "<|python_tag|>") == "llama_json"
    assert T.derive_tool_format(None, "a template without tools") is None

    class Tok:                       # a tokenizer whose template renders the probe call as XML
        def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=False, **kw):
            call = messages[-1]["tool_calls"][0]["function"]
            return f"<tool_call>\n<function={call['name']}>\n<parameter=k>\nv\n</parameter>\n</function>\n</tool_call>"

    assert T.derive_tool_format(Tok()) == "qwen_xml"
    assert T.tool_openers_closers(None, "mistral") == (["[TOOL_CALLS]"], [])
    assert T.tool_openers_closers(None, "gemma") == (["<|tool_call>"], ["<tool_call|>"])


def test_untyped_formats_take_their_types_from_the_schema():
    text = ("I will run it.<tool_call>\n<function=run>\n<parameter=command>\ntrue\n</parameter>\n"
            "<parameter=timeout_s>\n120\n</parameter>\n<parameter=local>\nfalse\n</parameter>\n</function>\n</tool_call>")
    content, calls = T.parse_tool_calls(text, TOOLS)
    assert content == "I will run it." and calls[0]["function"]["name"] == "run"
    # the declared string stays the four characters a shell needs; the declared integer / boolean convert
    assert _args(calls[0]) == {"command": "true", "timeout_s": 120, "local": False}
    # with no schema only the unambiguous cases convert
    assert T.coerce("123") == "123" and T.coerce("true") is True and T.coerce("[1, 2]") == [1, 2]
    assert T.coerce('"a b"') == '"a b"' and T.coerce("[1, 2]", "string") == "[1, 2]"


def test_every_wire_format_parses():
    cases = {
        "json": '<tool_call>\n{"name": "web_search", "arguments": {"query": "b200", "limit": 3}}\n</tool_call>',
        "zaya_inline": "<zyphra_tool_call><function=web_search(query='b200', limit=3)></zyphra_tool_call>",
        "atem": ('<atem:function_calls>\n<atem:invoke name="web_search">\n<atem:parameter name="query">b200'
                 '</atem:parameter>\n<atem:parameter name="limit">3</atem:parameter>\n</atem:invoke>\n'
                 "</atem:function_calls>"),
        "gemma": '<|tool_call>call:web_search{query:<|"|>b200<|"|>,limit:3}<tool_call|>',
        "laguna": "<tool_call>web_search<arg_key>query</arg_key><arg_value>b200</arg_value>"
                  "<arg_key>limit</arg_key><arg_value>3</arg_value></tool_call>",
        "mistral": '[TOOL_CALLS][{"name": "web_search", "arguments": {"query": "b200", "limit": 3}}]',
        "llama": '<|python_tag|>{"name": "web_search", "parameters": {"query": "b200", "limit": 3}}',
    }
    for name, text in cases.items():
        content, calls = T.parse_tool_calls(text, TOOLS)
        assert len(calls) == 1 and calls[0]["function"]["name"] == "web_search", name
        assert _args(calls[0]) == {"query": "b200", "limit": 3}, name
        assert calls[0]["id"].startswith("call_") and not content, name
    content, calls = T.parse_tool_calls('[web_search(query="b200", limit=3), run(command="ls")]', TOOLS, "pythonic")
    assert [c["function"]["name"] for c in calls] == ["web_search", "run"] and _args(calls[1]) == {"command": "ls"}
    # nested values in the Gemma syntax: bare keys at every depth, '<' allowed inside a string
    name, args = T.parse_gemma_call('call:run{command:<|"|>ls <dir> | wc<|"|>,env:{A:<|"|>1<|"|>,deep:{b:true}},n:[1,2]}')
    assert name == "run" and args == {"command": "ls <dir> | wc", "env": {"A": "1", "deep": {"b": True}}, "n": [1, 2]}
    # a body that is not a call stays visible instead of becoming a call named after its junk
    text = "<tool_call>call:bad{x:someBareword</tool_call>"
    assert T.parse_tool_calls(text, TOOLS) == (text, [])
    # two calls in one reply, text in between kept
    two = cases["json"] + " and then " + cases["json"].replace("b200", "h100")
    content, calls = T.parse_tool_calls(two, TOOLS)
    assert content == "and then" and [_args(c)["query"] for c in calls] == ["b200", "h100"]


def test_unknown_function_names_are_forwarded_unless_dropping_is_on(monkeypatch):
    text = '<tool_call>{"name": "web_fetch", "arguments": {}}</tool_call>'
    T.UNKNOWN_TOOL_SEEN.clear()
    _, calls = T.parse_tool_calls(text, TOOLS)
    assert [c["function"]["name"] for c in calls] == ["web_fetch"] and T.UNKNOWN_TOOL_SEEN == {"web_fetch": 1}
    monkeypatch.setenv("MSGL_DROP_UNKNOWN_TOOLS", "1")
    _, calls = T.parse_tool_calls(text, TOOLS)
    assert calls == [] and T.UNKNOWN_TOOL_SEEN == {"web_fetch": 2}


def test_forced_call_grammars_follow_the_format():
    xgr = pytest.importorskip("xgrammar")
    assert T.grammar_from_tools(TOOLS, "auto", "qwen_xml") is None
    info = xgr.TokenizerInfo([bytes([i]) for i in range(256)] + [b"<eos>"], vocab_size=257, stop_token_ids=[256])
    comp = xgr.GrammarCompiler(info)

    def accepts(spec, text):
        compiled = comp.compile_grammar(spec[5:]) if spec.startswith("ebnf:") else comp.compile_json_schema(spec)
        m = xgr.GrammarMatcher(compiled)
        return all(m.accept_token(b) for b in text.encode()) and m.accept_token(256)

    forced = {"type": "function", "function": {"name": "web_search"}}
    xml = T.grammar_from_tools(TOOLS, forced, "qwen_xml")
    good = "<tool_call>\n<function=web_search>\n<parameter=query>\nb200\n</parameter>\n</function>\n</tool_call>"
    assert xml.startswith("ebnf:") and accepts(xml, good)
    assert not accepts(xml, good.replace("web_search", "run"))          # the forced name only
    assert not accepts(xml, good.replace("query", "nonsense"))          # declared parameters only
    assert accepts(T.grammar_from_tools(TOOLS, "required", "qwen_xml"), good.replace("web_search", "run")
                   .replace("query", "command"))
    zaya = T.grammar_from_tools(TOOLS, forced, "zaya_xml")
    assert accepts(zaya, good.replace("<tool_call>", "<zyphra_tool_call>").replace("</tool_call>", "</zyphra_tool_call>"))
    gem = T.grammar_from_tools(TOOLS, forced, "gemma")
    assert accepts(gem, '<|tool_call>call:web_search{query:<|"|>a < b<|"|>,limit:3}<tool_call|>')
    assert not accepts(gem, '<|tool_call>call:web_search{"query":"x"}<tool_call|>')
    atem = T.grammar_from_tools(TOOLS, forced, "atem")
    assert accepts(atem, '<atem:function_calls>\n<atem:invoke name="web_search">\n<atem:parameter name="limit">3'
                         "</atem:parameter>\n</atem:invoke>\n</atem:function_calls>")
    js = T.grammar_from_tools(TOOLS, forced, "json")
    assert accepts(js, '{"name": "web_search", "arguments": {"query": "x", "limit": 2}}')
    assert not accepts(js, '{"name": "run", "arguments": {}}')
    # every parsed result of a grammar-conforming call is a call the parser understands
    assert T.parse_tool_calls(good, TOOLS)[1][0]["function"]["name"] == "web_search"


def test_tools_with_their_own_defs_do_not_collide():
    tools = [{"type": "function", "function": {"name": f"t{i}", "parameters": {
        "type": "object", "properties": {"p": {"$ref": "#/$defs/P"}}, "$defs": {"P": {"type": kind}}}}}
        for i, kind in enumerate(("string", "integer"))]
    schema = json.loads(T.grammar_from_tools(tools, "required", "json"))
    assert set(schema["$defs"]) == {"t0__P", "t1__P"}
    refs = [v["properties"]["arguments"]["properties"]["p"]["$ref"] for v in schema["anyOf"]]
    assert refs == ["#/$defs/t0__P", "#/$defs/t1__P"]
    tag = json.loads(T.structural_tag_for_tools(TOOLS, "json")[len("structural_tag:"):])
    assert tag["triggers"] == ["<tool_call>"] and len(tag["structures"]) == 2
    assert T.structural_tag_for_tools(TOOLS, "qwen_xml") is None


def test_streaming_json_call_streams_name_then_argument_text():
    text = 'Sure.<tool_call>\n{"name": "web_search", "arguments": {"query": "b200 specs", "limit": 3}}\n</tool_call> done'
    for step in (1, 3, 7, 1000):
        st = T.ToolCallStreamState(TOOLS, "json")
        content, deltas = "", []
        for i in range(0, len(text), step):
            c, d = st.push(text[i:i + step])
            content += c
            deltas += d
        c, d = st.flush()
        content += c
        deltas += d
        assert content == "Sure. done", (step, content)
        heads = [x for x in deltas if "id" in x]
        assert len(heads) == 1 and heads[0]["function"]["name"] == "web_search" and heads[0]["index"] == 0
        joined = "".join(x["function"]["arguments"] for x in deltas)
        assert json.loads(joined) == {"query": "b200 specs", "limit": 3}, (step, joined)
        if step == 1:
            assert len(deltas) > 5          # the arguments arrived in pieces, not in one burst


def test_streaming_holds_other_bodies_until_their_closer_and_recovers_at_the_end():
    xml = ("<tool_call>\n<function=run>\n<parameter=command>\nls -la\n</parameter>\n</function>\n</tool_call>"
           "<tool_call>\n<function=web_search>\n<parameter=limit>\n2\n</parameter>\n</function>\n</tool_call>")
    st = T.ToolCallStreamState(TOOLS, "qwen_xml")
    got = []
    for i in range(0, len(xml), 4):
        c, d = st.push(xml[i:i + 4])
        assert c == ""
        got += d
    assert [(x["index"], x["function"]["name"]) for x in got] == [(0, "run"), (1, "web_search")]
    assert _args(got[1]) == {"limit": 2}
    # an opener split across deltas is held back, not leaked as content
    st = T.ToolCallStreamState(TOOLS, "json")
    assert st.push("text <tool_")[0] == "text " and st.held_chars == len("<tool_")
    assert st.push("box> more")[0] == "<tool_box> more"
    # a call cut off by the token limit still yields what it holds
    st = T.ToolCallStreamState(TOOLS, "qwen_xml")
    st.push("<tool_call>\n<function=run>\n<parameter=command>\nls\n</parameter>\n")
    rest, calls = st.flush()
    assert rest == "" and calls[0]["function"]["name"] == "run" and _args(calls[0]) == {"command": "ls"}
    # no call at all: everything is content
    st = T.ToolCallStreamState(TOOLS, "json")
    assert st.push("plain answer")[0] + st.flush()[0] == "plain answer" and st.flush()[1] == []
