"""Streaming reply parser: reasoning / content split, Qwen XML and JSON and DSML tool calls, streamed argument pieces,
lenient JSON and typed values. Every case is also run cut into 1-, 3- and 7-character pieces: the result may not
depend on the cut. Behaviours follow the reference's parser tests (`crates/fe-server/src/parser.rs:1100-1510`)."""
import json
import random

import pytest

from ferrite_b200.server.parser import StreamParser, lenient_json, merge_tool_calls, strip_trailing_commas, typed_value
from ferrite_b200.server.toolcall import ForcedCall, ToolSet

TOOLS = [
    {"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {
        "location": {"type": "string"}, "days": {"type": "integer"}, "metric": {"type": "boolean"}}}}},
    {"type": "function", "function": {"name": "search", "parameters": {"type": "object", "properties": {
        "query": {"type": "string"}, "limit": {"type": "number"}, "tags": {"type": "array", "items": {"type": "string"}}}}}},
    {"type": "function", "function": {"name": "write", "parameters": {"type": "object", "properties": {
        "path": {"type": "string"}, "content": {"type": "string"}, "edits": {"type": "array"}}}}},
]


def run(text, thinking=False, tools=True, step=None, **kw):
    p = StreamParser(ToolSet(TOOLS) if tools else None, thinking=thinking, **kw)
    reasoning, content, calls = "", "", []
    pieces = [text] if step is None else [text[i:i + step] for i in range(0, len(text), step)]
    for piece in pieces:
        d = p.push(piece)
        reasoning += d.reasoning
        content += d.content
        calls += d.tool_calls
    d = p.finish()
    reasoning += d.reasoning
    content += d.content
    calls += d.tool_calls
    merged = [(c["function"]["name"], json.loads(c["function"]["arguments"])) for c in merge_tool_calls(calls)]
    return reasoning, content, merged


def parse(text, **kw):
    whole = run(text, **kw)
    for step in (1, 3, 7):
        assert run(text, step=step, **kw) == whole, f"pieces of {step} changed the result of {text!r}"
    return whole


def test_reasoning_then_content_and_thinking_off():
    assert parse("Let me think.\nOK.\n</think>\n\nThe answer is 4.", thinking=True, tools=False) == ("Let me think.\nOK.", "The answer is 4.", [])
    assert parse("All of this is content.", tools=False) == ("", "All of this is content.", [])
    assert parse("never closed", thinking=True, tools=False) == ("never closed", "", [])
    assert parse("<think>\nhm\n</think>\n\nhi", tools=False) == ("hm", "hi", [])


def test_content_keeps_inner_whitespace_and_angle_brackets():
    r, c, _ = parse("r</think>\n\n```rust\nfn a() -> Vec<u8> {\n    vec![]\n}\n```\n", thinking=True, tools=False)
    assert r == "r" and c == "```rust\nfn a() -> Vec<u8> {\n    vec![]\n}\n```\n"
    assert parse("a < b and c > d <x> </y>", tools=True)[1] == "a < b and c > d <x> </y>"


def test_think_only_opens_at_the_start_of_content():
    assert parse("OK<think>x</think>y", tools=False) == ("", "OK<think>xy", [])
    assert parse("  <think>x</think>y", tools=False) == ("x", "y", [])


def test_single_and_parallel_tool_calls_with_typed_values():
    text = ("I should check.\n</think>\n\n<tool_call>\n<function=get_weather>\n<parameter=location>\nParis\n</parameter>\n"
            "<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>")
    assert parse(text, thinking=True) == ("I should check.", "", [("get_weather", {"location": "Paris", "days": 3})])
    text = ("Let me look both up.\n\n<tool_call>\n<function=get_weather>\n<parameter=location>\nOslo\n</parameter>\n"
            "<parameter=metric>\ntrue\n</parameter>\n</function>\n</tool_call>\n<tool_call>\n<function=search>\n"
            "<parameter=query>\nbest café in Oslo\n</parameter>\n<parameter=limit>\n2.5\n</parameter>\n</function>\n</tool_call>")
    assert parse(text) == ("", "Let me look both up.", [("get_weather", {"location": "Oslo", "metric": True}),
                                                        ("search", {"query": "best café in Oslo", "limit": 2.5})])


def test_call_inside_reasoning_ends_it_but_quoted_markup_does_not():
    text = "need weather\n<tool_call>\n<function=get_weather>\n<parameter=location>\nRome\n</parameter>\n</function>\n</tool_call>"
    assert parse(text, thinking=True) == ("need weather", "", [("get_weather", {"location": "Rome"})])
    quoted = "The content is `<tool_call><function=x><parameter=y>1</parameter></function></tool_call> <div>` literally."
    text = quoted + "\n</think>\n\n<tool_call>\n<function=search>\n<parameter=query>\nq\n</parameter>\n</function>\n</tool_call>"
    assert parse(text, thinking=True) == (quoted, "", [("search", {"query": "q"})])
    assert parse("thinking <tool_call>", thinking=True) == ("thinking", "", [])


def test_tools_off_leaves_markup_in_content():
    text = "<tool_call>\n<function=search>\n<parameter=query>\nx\n</parameter>\n</function>\n</tool_call>"
    assert parse(text, tools=False) == ("", text, [])


def test_bare_function_two_functions_in_one_block_and_cut_off_call():
    assert parse("<function=search>\n<parameter=query>\na\n</parameter>\n</function>\nmore text") == \
        ("", "more text", [("search", {"query": "a"})])
    text = ("<tool_call>\n<function=search>\n<parameter=query>\na\n</parameter>\n</function>\n<function=search>\n"
            "<parameter=query>\nb\n</parameter>\n</function>\n</tool_call>")
    assert parse(text)[2] == [("search", {"query": "a"}), ("search", {"query": "b"})]
    assert parse("<tool_call>\n<function=search>\n<parameter=query>\nhalf a que")[2] == [("search", {"query": "half a que"})]
    assert parse("<tool_call>\n<function=get_weather>\n</function>\n</tool_call>")[2] == [("get_weather", {})]


def test_json_body_and_lenient_forms():
    assert parse('<tool_call>\n{"name": "search", "arguments": {"query": "q"}}\n</tool_call>')[2] == [("search", {"query": "q"})]
    assert parse('<tool_call>\n{"name": "search", "arguments": {"query": "q", "limit": "3",},}\n</tool_call>')[2] == \
        [("search", {"query": "q", "limit": 3.0})]
    assert parse('<tool_call>\n```json\n{"name": "search", "arguments": "{\\"query\\": \\"q\\"}"}\n```\n</tool_call>')[2] == \
        [("search", {"query": "q"})]
    assert parse('<tool_call>\n{"name": "search", "arguments": {"query": "cut off')[2] == [("search", {"query": "cut off"})]


def test_parallel_calls_off_keeps_the_first():
    text = ("<tool_call>\n<function=search>\n<parameter=query>\na\n</parameter>\n</function>\n</tool_call>\n<tool_call>\n"
            "<function=search>\n<parameter=query>\nb\n</parameter>\n</function>\n</tool_call>")
    assert parse(text, max_tool_calls=1)[2] == [("search", {"query": "a"})]


def test_block_that_is_not_a_call_is_given_back_verbatim():
    assert parse("Use <tool_call>\nnot json here</tool_call> ok") == ("", "Use <tool_call>\nnot json here</tool_call> ok", [])
    assert parse("Use <tool_call>\nunclosed") == ("", "Use <tool_call>\nunclosed", [])


def test_streaming_emits_the_name_first_then_argument_pieces():
    p = StreamParser(ToolSet(TOOLS))
    d = p.push("Checking.\n\n<tool_call>\n<function=search>\n<parameter=query>\nab")
    assert d.content == "Checking."
    assert d.tool_calls[0]["function"]["name"] == "search" and d.tool_calls[0]["id"] and d.tool_calls[0]["type"] == "function"
    assert "".join(t["function"]["arguments"] for t in d.tool_calls) == '{"query": "ab'
    d = p.push("c\n</parameter>\n</function>\n</tool_call>")
    assert "".join(t["function"]["arguments"] for t in d.tool_calls) == 'c"}' and all("id" not in t for t in d.tool_calls)
    assert p.finish().empty()
    # a long string value arrives in many pieces; a non-string value in one, when it is complete
    p = StreamParser(ToolSet(TOOLS))
    n_pieces = 0
    text = "<tool_call>\n<function=write>\n<parameter=content>\n" + "line of text\n" * 50 + "</parameter>\n<parameter=edits>\n[1, 2,\n 3]\n</parameter>\n</function>\n</tool_call>"
    calls = []
    for i in range(0, len(text), 40):
        d = p.push(text[i:i + 40])
        n_pieces += sum(1 for t in d.tool_calls if t["function"].get("arguments"))
        calls += d.tool_calls
    calls += p.finish().tool_calls
    args = json.loads(merge_tool_calls(calls)[0]["function"]["arguments"])
    assert args == {"content": "line of text\n" * 49 + "line of text", "edits": [1, 2, 3]} and n_pieces > 10


def test_values_keep_inner_newlines_and_markup_lookalikes():
    text = "<tool_call>\n<function=write>\n<parameter=content>\n<div>\n  a < b\n\n</div>\n</parameter>\n</function>\n</tool_call>"
    assert parse(text)[2] == [("write", {"content": "<div>\n  a < b\n\n</div>"})]
    # a parameter whose closing tag is missing ends at the next marker
    text = "<tool_call>\n<function=search>\n<parameter=query>\nabc\n<parameter=limit>\n4\n</function>\n</tool_call>"
    assert parse(text)[2] == [("search", {"query": "abc", "limit": 4})]


def test_forced_openers():
    any_call, named = ForcedCall.make(None), ForcedCall.make("search")
    assert any_call.opener == "<tool_call>\n<function=" and named.opener == "<tool_call>\n<function=search>\n"
    assert run("get_weather>\n<parameter=location>\nRome\n</parameter>\n</function>\n</tool_call>", prefix=any_call.opener)[2] == \
        [("get_weather", {"location": "Rome"})]
    assert run("<parameter=query>\nx\n</parameter>\n</function>\n</tool_call>", prefix=named.opener)[2] == [("search", {"query": "x"})]
    assert ForcedCall.make("f", dsml=True).opener.endswith('<｜DSML｜ invoke name="f">\n')


# ---- DSML ----------------------------------------------------------------------------------------------------------

def dcall(name, body):
    return f'<｜DSML｜ invoke name="{name}">\n{body}</｜DSML｜ invoke>\n'


def sp(name, v, string=True):
    return f'<｜DSML｜ parameter name="{name}" string="{"true" if string else "false"}">{v}</｜DSML｜ parameter>\n'


def test_dsml_calls():
    text = "Looking.\n\n<｜DSML｜ calls>\n" + dcall("search", sp("query", "rust") + sp("limit", "3", False)) + \
        dcall("get_weather", sp("location", "Oslo")) + "</｜DSML｜ calls>"
    assert parse(text, dsml=True) == ("", "Looking.", [("search", {"query": "rust", "limit": 3.0}), ("get_weather", {"location": "Oslo"})])
    # the opening calls tag is missing; an invoke is missing its closing tags
    assert parse(dcall("search", sp("query", "a")), dsml=True)[2] == [("search", {"query": "a"})]
    text = '<｜DSML｜ calls>\n<｜DSML｜ invoke name="search">\n<｜DSML｜ parameter name="query" string="true">half'
    assert parse(text, dsml=True)[2] == [("search", {"query": "half"})]
    # schema types win over the string attribute; arrays in any of their written forms
    text = "<｜DSML｜ calls>\n" + dcall("search", sp("limit", "7", True) + sp("tags", '["a", "b",]', False)) + "</｜DSML｜ calls>"
    assert parse(text, dsml=True)[2] == [("search", {"limit": 7.0, "tags": ["a", "b"]})]
    # values with markup inside
    text = "<｜DSML｜ calls>\n" + dcall("write", sp("content", "<b>x</b>\n<｜DSML｜ not a tag\n")) + "</｜DSML｜ calls>"
    assert parse(text, dsml=True)[2] == [("write", {"content": "<b>x</b>\n<｜DSML｜ not a tag"})]
    # XML markup is plain text for a DSML parser
    assert parse("<tool_call>x</tool_call>", dsml=True)[1] == "<tool_call>x</tool_call>"


def test_lenient_json_and_typed_values():
    assert strip_trailing_commas('{"a": [1, 2, ], "b": ",}" , }') == '{"a": [1, 2 ], "b": ",}"  }'
    assert lenient_json('```json\n{"a": 1}\n```') == (True, {"a": 1})
    assert lenient_json('"{\\"a\\": [1]}"') == (True, {"a": [1]})
    assert lenient_json('{"a": {"b": [1, 2') == (True, {"a": {"b": [1, 2]}})
    assert lenient_json("not json")[0] is False
    assert typed_value("12", {"type": "integer"}) == 12 and typed_value("12", {"type": "string"}) == "12"
    assert typed_value("yes", {"type": "integer"}) == "yes"
    assert typed_value("[1, 2]", None) == [1, 2] and typed_value("plain", None) == "plain"
    assert typed_value('{"k": "3"}', {"type": "object", "properties": {"k": {"type": "integer"}}}) == {"k": 3}


def test_random_cuts_never_change_the_result():
    pieces = ["hi", " ", "\n", "é🦀", "<", ">", "<think>", "</think>", "<tool_call>", "</tool_call>", "<function=search>",
              "<function=get_weather>", "<parameter=query>", "<parameter=days>", "</parameter>", "</function>",
              '{"name": "search", "arguments": {}}', "3", "<tool", "</fun"]
    rng = random.Random(3)
    for case in range(600):
        text = "".join(rng.choice(pieces) for _ in range(rng.randint(1, 14)))
        kw = dict(thinking=case % 2 == 0, tools=case % 4 < 2)
        whole = run(text, **kw)
        for step in (1, 3, 7):
            assert run(text, step=step, **kw) == whole, (text, step)
        p = StreamParser(ToolSet(TOOLS) if kw["tools"] else None, thinking=kw["thinking"])
        acc = ["", "", []]
        i = 0
        while i < len(text):
            k = rng.randint(1, 5)
            d = p.push(text[i:i + k])
            acc[0] += d.reasoning; acc[1] += d.content; acc[2] += d.tool_calls
            i += k
        d = p.finish()
        acc[0] += d.reasoning; acc[1] += d.content; acc[2] += d.tool_calls
        got = (acc[0], acc[1], [(c["function"]["name"], json.loads(c["function"]["arguments"])) for c in merge_tool_calls(acc[2])])
        assert got == whole, text


def test_model_opened_think_itself_inside_an_open_block():
    assert parse("<think>\nhm\n</think>\n\nhi", thinking=True, tools=False) == ("hm", "hi", [])
