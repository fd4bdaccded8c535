"""Chat template rendering (Jinja, Hugging Face conventions) with a built-in ChatML template that knows tools
and thinking. Counterpart of `crates/fe-server/src/template.rs` (minijinja render matching HF byte for byte)."""
from __future__ import annotations

import datetime
import json
import os
from typing import Any, Dict, List, Optional

import jinja2
from jinja2.sandbox import ImmutableSandboxedEnvironment


DEFAULT_TEMPLATE = r"""{%- if tools %}
{{- '<|im_start|>system\n' }}
{%- if messages[0].role == 'system' %}{{- messages[0].content + '\n\n' }}{%- endif %}
{{- "# Tools\n\nYou have access to the following functions:\n\n<tools>" }}
{%- for tool in tools %}{{- "\n" }}{{- tool | tojson }}{%- endfor %}
{{- "\n</tools>\n\nTo call a function, reply in exactly this format and nothing after it:\n\n<tool_call>\n<function=function_name>\n<parameter=parameter_name>\nvalue\n</parameter>\n</function>\n</tool_call>\n\nGive every required parameter. A value may span several lines. Explain before the call, never after it.<|im_end|>\n" }}
{%- else %}
{%- if messages[0].role == 'system' %}{{- '<|im_start|>system\n' + messages[0].content + '<|im_end|>\n' }}{%- endif %}
{%- endif %}
{%- for message in messages %}
{%- if message.role == 'system' and loop.first %}
{%- elif message.role == 'assistant' %}
{{- '<|im_start|>assistant\n' }}
{%- if message.reasoning_content %}{{- '<think>\n' + message.reasoning_content + '\n</think>\n\n' }}{%- endif %}
{%- if message.content %}{{- message.content }}{%- endif %}
{%- for tc in message.tool_calls or [] %}
{%- if message.content or not loop.first %}{{- '\n' }}{%- endif %}
{{- '<tool_call>\n<function=' + tc.function.name + '>\n' }}
{%- if tc.function.arguments is mapping %}
{%- for k, v in tc.function.arguments | items %}
{{- '<parameter=' + k + '>\n' }}
{%- if v is string %}{{- v }}{%- else %}{{- v | tojson }}{%- endif %}
{{- '\n</parameter>\n' }}
{%- endfor %}
{%- endif %}
{{- '</function>\n</tool_call>' }}
{%- endfor %}
{{- '<|im_end|>\n' }}
{%- elif message.role == 'tool' %}
{{- '<|im_start|>user\n<tool_response>\n' + message.content + '\n</tool_response><|im_end|>\n' }}
{%- else %}
{{- '<|im_start|>' + message.role + '\n' + message.content + '<|im_end|>\n' }}
{%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
{{- '<|im_start|>assistant\n' }}
{%- if enable_thinking is defined and enable_thinking is false %}{{- '<think>\n\n</think>\n\n' }}{%- endif %}
{%- endif %}"""


def _raise(msg):
    raise jinja2.TemplateError(msg)


def _content_text(c: Any) -> str:
    """OpenAI content may be a list of parts; templates want text."""
    if c is None:
        return ""
    if isinstance(c, str):
        return c
    if isinstance(c, list):
        return "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type", "text") == "text")
    return str(c)


class ChatTemplate:
    def __init__(self, source: Optional[str] = None):
        self.env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
        self.env.filters["tojson"] = lambda v, indent=None, ensure_ascii=False: json.dumps(v, indent=indent, ensure_ascii=ensure_ascii)
        self.env.globals["raise_exception"] = _raise
        self.env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        self.source = source or DEFAULT_TEMPLATE
        self.tpl = self.env.from_string(self.source)

    @staticmethod
    def from_dir(model_dir: Optional[str]) -> "ChatTemplate":
        if model_dir:
            p = os.path.join(model_dir, "chat_template.jinja")
            if os.path.exists(p):
                return ChatTemplate(open(p).read())
            p = os.path.join(model_dir, "tokenizer_config.json")
            if os.path.exists(p):
                t = json.load(open(p)).get("chat_template")
                if isinstance(t, str):
                    return ChatTemplate(t)
        return ChatTemplate(None)

    def render(self, messages: List[Dict[str, Any]], tools: Optional[List[Dict[str, Any]]] = None,
               add_generation_prompt: bool = True, **kwargs) -> str:
        msgs = []
        for m in messages:
            mm = dict(m)
            mm["content"] = _content_text(m.get("content"))
            if mm.get("tool_calls"):
                tcs = []
                for tc in mm["tool_calls"]:
                    tc = json.loads(json.dumps(tc))
                    args = tc.get("function", {}).get("arguments")
                    if isinstance(args, str):
                        try:
                            tc["function"]["arguments"] = json.loads(args)
                        except Exception:
                            pass
                    tcs.append(tc)
                mm["tool_calls"] = tcs
            msgs.append(mm)
        return self.tpl.render(messages=msgs, tools=tools or None, add_generation_prompt=add_generation_prompt, **kwargs)
