"""Writes `tests/fixtures/hf_template_refs.json`: renders of chat templates by Hugging Face `transformers`' own template
engine, which `ChatTemplate.render` must reproduce byte for byte (the reference checks its minijinja renderer against
the same kind of file, `crates/fe-server/tests/template_hf.rs` + `tools/gen_template_refs.py`).

    python -m ferrite_b200.server.gen_template_refs tests/fixtures/hf_template_refs.json

Each case holds the template source (the built-in one, and a second one that exercises namespace(), loop controls,
`tojson(indent=...)`, non-ASCII text, whitespace control and `raise_exception`), the messages / tools / keyword
arguments, and the text `transformers` produced (or the fact that it raised).
"""
from __future__ import annotations

import json
import sys

from .template import DEFAULT_TEMPLATE

SECOND_TEMPLATE = r"""{%- set ns = namespace(last_user=-1, n_tools=0) %}
{%- for m in messages %}
    {%- if m.role == 'user' %}{%- set ns.last_user = loop.index0 %}{%- endif %}
{%- endfor %}
{%- if tools %}
    {{- '[TOOLS]' + (tools | tojson(indent=2)) + '[/TOOLS]\n' }}
    {%- for t in tools %}{%- set ns.n_tools = ns.n_tools + 1 %}{%- endfor %}
{%- endif %}
{%- for m in messages %}
    {%- if m.role not in ['system', 'user', 'assistant', 'tool'] %}
        {{- raise_exception('unknown role ' + m.role) }}
    {%- endif %}
    {%- if m.role == 'tool' and ns.n_tools == 0 %}{%- continue %}{%- endif %}
    {{- '<' + m.role + (' last' if loop.index0 == ns.last_user else '') + '>' }}
    {%- if m.content is string %}
        {{- m.content | trim }}
    {%- endif %}
    {%- if m.tool_calls %}
        {%- for tc in m.tool_calls %}
            {{- '\n[CALL ' ~ loop.index ~ '/' ~ loop.length ~ '] ' + tc.function.name + ' ' + (tc.function.arguments | tojson) }}
        {%- endfor %}
    {%- endif %}
    {{- '</' + m.role + '>\n' }}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<assistant>' }}{% if style is defined %}{{ '(' + style | upper + ')' }}{% endif %}
{%- endif %}
"""

TOOLS = [
    {"type": "function", "function": {"name": "get_weather", "description": "Weather for a city — with “quotes” & <tags>",
                                      "parameters": {"type": "object", "properties": {"city": {"type": "string"},
                                                                                       "days": {"type": "integer", "default": 3}},
                                                     "required": ["city"]}}},
    {"type": "function", "function": {"name": "noop", "parameters": {"type": "object", "properties": {}}}},
]

CONVS = {
    "plain": [{"role": "user", "content": "Hello"}],
    "system_multi_turn": [{"role": "system", "content": "You are terse."}, {"role": "user", "content": "2+2?"},
                          {"role": "assistant", "content": "4"}, {"role": "user", "content": "  and 3+3?\n"}],
    "unicode": [{"role": "user", "content": "naïve café ☕ 日本語 \"quoted\" \\ backslash\ttab"}],
    "reasoning": [{"role": "user", "content": "why?"},
                  {"role": "assistant", "content": "Because.", "reasoning_content": "Think.\nTwice."},
                  {"role": "user", "content": "ok"}],
    "tool_round_trip": [
        {"role": "system", "content": "Use tools."}, {"role": "user", "content": "Weather in Oslo?"},
        {"role": "assistant", "content": "", "tool_calls": [
            {"id": "call_1", "type": "function", "function": {"name": "get_weather", "arguments": {"city": "Oslo", "days": 2}}},
            {"id": "call_2", "type": "function", "function": {"name": "get_weather", "arguments": {"city": "Bergen", "opts": {"a": [1, 2.5, None, True]}}}}]},
        {"role": "tool", "content": "{\"temp\": -3}"}, {"role": "tool", "content": "{\"temp\": 4}"},
        {"role": "user", "content": "thanks"}],
    "call_with_text": [{"role": "user", "content": "go"},
                       {"role": "assistant", "content": "Checking.", "tool_calls": [
                           {"id": "c", "type": "function", "function": {"name": "noop", "arguments": {}}}]},
                       {"role": "tool", "content": "done"}],
}


def cases():
    out = []
    for tname, tsrc in (("default", DEFAULT_TEMPLATE), ("second", SECOND_TEMPLATE)):
        for cname, conv in CONVS.items():
            for tools in (None, TOOLS):
                for gen in (True, False):
                    for kw in ({}, {"enable_thinking": False}, {"style": "brief"}):
                        if kw and not gen:
                            continue
                        out.append({"template": tname, "conversation": cname, "messages": conv, "tools": tools,
                                    "add_generation_prompt": gen, "kwargs": kw})
        out.append({"template": tname, "conversation": "bad_role", "messages": [{"role": "robot", "content": "x"}], "tools": None,
                    "add_generation_prompt": True, "kwargs": {}})
    return out


def main() -> int:
    from transformers.utils.chat_template_utils import render_jinja_template
    import transformers
    path = sys.argv[1] if len(sys.argv) > 1 else "tests/fixtures/hf_template_refs.json"
    src = {"default": DEFAULT_TEMPLATE, "second": SECOND_TEMPLATE}
    done = []
    for c in cases():
        try:
            text = render_jinja_template([c["messages"]], tools=c["tools"], chat_template=src[c["template"]],
                                         add_generation_prompt=c["add_generation_prompt"], **c["kwargs"])
            text = text[0][0] if isinstance(text, tuple) else text[0]
            done.append({**c, "expected": text})
        except Exception as e:                                       # noqa: BLE001
            done.append({**c, "raises": type(e).__name__})
    with open(path, "w") as f:
        json.dump({"transformers": transformers.__version__, "templates": src, "cases": done}, f, ensure_ascii=False, indent=1)
    print(f"{len(done)} cases -> {path}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
