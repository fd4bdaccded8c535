"""Streaming reply parser: reasoning, content and tool calls out of model text that arrives in arbitrary pieces.

What it recognises (the behaviours of the reference's `crates/fe-server/src/parser.rs`):

* `<think>...</think>`: with `thinking=True` the reply starts as reasoning and `</think>` switches to content; a
  `<think>` the model writes itself opens reasoning only at the very start of the content; a later `</think>` is dropped;
* Qwen XML tool calls: `<tool_call>\\n<function=NAME>\\n<parameter=KEY>\\nVALUE\\n</parameter>...</function>\\n</tool_call>`,
  several `<function=` in one block, a bare `<function=` without the block, and a `<tool_call>` inside the reasoning
  (the model's own opener is followed by a newline; quoted markup in prose is not) as an implicit end of thinking;
* a JSON body inside `<tool_call>` (`{"name": .., "arguments": {..}}`), read leniently: code fences, trailing commas,
  a missing closing brace, double-encoded arguments;
* DeepSeek DSML calls: `<｜DSML｜ calls>` / `<｜DSML｜ invoke name="F">` / `<｜DSML｜ parameter name="p" string="true|false">`;
* a forced opener (`tool_choice` required / named): the reply starts inside the call.

Tool calls stream: the name goes out as soon as it is complete (a delta with `id`, `type`, `function.name`), then the
arguments as pieces of JSON text whose concatenation is the complete arguments object; a string parameter streams
while it is written, any other type is converted (by the tool's JSON schema, else by its looks) when its value ends.
A block that turns out not to be a call is given back to the content verbatim. Text that could still become a marker
is held back, so the result never depends on how the text was cut into pieces.
"""
from __future__ import annotations

import json
import re
import zlib
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .toolcall import ToolSet, coerce

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
CALL_OPEN, CALL_CLOSE = "<tool_call>", "</tool_call>"
FUNC_OPEN, FUNC_CLOSE = "<function=", "</function>"
PARAM_OPEN, PARAM_CLOSE = "<parameter=", "</parameter>"
DS_CALLS, DS_CALLS_END = "<｜DSML｜ calls>", "</｜DSML｜ calls>"
DS_INVOKE, DS_INVOKE_END = "<｜DSML｜ invoke name=\"", "</｜DSML｜ invoke>"
DS_PARAM, DS_PARAM_END = "<｜DSML｜ parameter name=\"", "</｜DSML｜ parameter>"


@dataclass
class Delta:
    reasoning: str = ""
    content: str = ""
    tool_calls: List[Dict[str, Any]] = field(default_factory=list)   # OpenAI tool_call delta objects

    def empty(self) -> bool:
        return not (self.reasoning or self.content or self.tool_calls)


def _holdback(buf: str, markers) -> int:
    """Length of the longest suffix of buf that is a proper prefix of one of the markers."""
    best = 0
    for t in markers:
        for k in range(min(len(t) - 1, len(buf)), best, -1):
            if buf.endswith(t[:k]):
                best = k
                break
    return best


def _find_first(buf: str, markers):
    pos, tag = -1, None
    for t in markers:
        i = buf.find(t)
        if i >= 0 and (pos < 0 or i < pos or (i == pos and len(t) > len(tag))):
            pos, tag = i, t
    return pos, tag


# ---- lenient JSON --------------------------------------------------------------------------------------------------

def strip_trailing_commas(t: str) -> str:
    """Remove commas that sit right before a closing bracket or brace (outside strings)."""
    out, in_str, esc = [], False, False
    for i, ch in enumerate(t):
        if in_str:
            out.append(ch)
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        if ch == ",":
            j = i + 1
            while j < len(t) and t[j] in " \t\r\n":
                j += 1
            if j < len(t) and t[j] in "]}":
                continue
        out.append(ch)
    return "".join(out)


def _close_open_brackets(t: str) -> str:
    """Append the closers a cut-off JSON text still needs (an open string, then brackets innermost first)."""
    stack, in_str, esc = [], False, False
    for ch in t:
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            stack.append("}" if ch == "{" else "]")
        elif ch in "}]" and stack:
            stack.pop()
    return t + ('"' if in_str else "") + "".join(reversed(stack))


def lenient_json(raw: str, depth: int = 0):
    """JSON as models write it: plain, inside a code fence, with trailing commas, cut off before its closing brackets, or
    double-encoded (a JSON string that holds JSON). Returns (ok, value)."""
    t = raw.strip()
    if t.startswith("```"):
        t = re.sub(r"^```[a-zA-Z0-9_-]*\s*", "", t)
        t = re.sub(r"\s*```\s*$", "", t)
    if not t:
        return False, None
    for cand in (t, strip_trailing_commas(t), _close_open_brackets(strip_trailing_commas(t))):
        try:
            v = json.loads(cand)
        except (json.JSONDecodeError, RecursionError):
            continue
        if isinstance(v, str) and depth < 2 and v.strip()[:1] in ("{", "["):
            ok, inner = lenient_json(v, depth + 1)
            if ok and isinstance(inner, (dict, list)):
                return True, inner
        return True, v
    # a JSON value followed by junk: the longest prefix that parses
    if t[:1] in "{[":
        dec = json.JSONDecoder()
        try:
            v, _ = dec.raw_decode(t)
            return True, v
        except json.JSONDecodeError:
            pass
    return False, None


def typed_value(raw: str, schema: Optional[Dict[str, Any]]):
    """A parameter value as the schema types it: strings stay as written; other types are read as (lenient) JSON and
    bent towards the schema; without a schema a value that parses as a JSON number / boolean / null / object / array
    is that, anything else a string."""
    t = schema.get("type") if isinstance(schema, dict) else None
    if isinstance(t, list):
        t = next((x for x in t if x != "null"), None)
    if t == "string":
        return raw
    ok, v = lenient_json(raw)
    if t is None:
        if ok and not isinstance(v, str):
            return v
        return raw
    if ok:
        return coerce(v, schema)
    return coerce(raw.strip(), schema)


def parse_call_body(body: str, tools: Optional[ToolSet]) -> Optional[Dict[str, Any]]:
    """Body of one `<tool_call>` as a whole (non-streaming helper): {"name", "arguments" (JSON text)} or None."""
    p = StreamParser(tools if tools is not None else ToolSet([]), accept_any_tool=True)
    d = p.push(CALL_OPEN + body + CALL_CLOSE)
    f = p.finish()
    calls = merge_tool_calls(d.tool_calls + f.tool_calls)
    if not calls:
        return None
    return {"name": calls[0]["function"]["name"], "arguments": calls[0]["function"]["arguments"]}


def merge_tool_calls(deltas: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """Fold streamed tool-call deltas (a start delta then argument pieces per index) into whole calls."""
    out: Dict[int, Dict[str, Any]] = {}
    for d in deltas:
        i = d["index"]
        if i not in out:
            out[i] = {"index": i, "id": d.get("id", ""), "type": "function", "function": {"name": "", "arguments": ""}}
        if d.get("id"):
            out[i]["id"] = d["id"]
        fn = d.get("function") or {}
        if fn.get("name"):
            out[i]["function"]["name"] = fn["name"]
        out[i]["function"]["arguments"] += fn.get("arguments", "")
    return [out[i] for i in sorted(out)]


def _jstr(s: str) -> str:
    """The inside of a JSON string literal for `s` (no quotes), so pieces can be streamed and concatenated."""
    return json.dumps(s, ensure_ascii=False)[1:-1]


class StreamParser:
    """Feed text with `push`, get `Delta`s; `finish` flushes what was held back and closes a cut-off call.

    thinking: the prompt ended inside an open `<think>` block. tools: a `ToolSet` (empty / None: call markup is plain
    content). max_tool_calls: later calls are parsed but not reported (`parallel_tool_calls: false` -> 1). dsml: DSML
    call syntax instead of the Qwen XML one. prefix: text the prompt was forced to end with (`ForcedCall.opener`), fed
    first so the reply continues inside the call."""

    def __init__(self, tools: Optional[ToolSet] = None, thinking: bool = False, prefix: str = "",
                 max_tool_calls: Optional[int] = None, dsml: bool = False, accept_any_tool: bool = False):
        self.tools = tools
        self.tools_on = bool(tools) or accept_any_tool
        self.dsml = dsml
        self.max_calls = max_tool_calls
        self.mode = "think" if thinking else "text"
        self.buf = ""
        self.n_calls = 0
        self.malformed = False
        self.started = {"think": False, "text": False}     # leading whitespace of each stream is dropped
        self.ws = {"think": "", "text": ""}                 # whitespace held until more text follows (dropped before a marker)
        self.text_seen = False                              # anything at all went to content (a late <think> is text)
        # call in progress
        self.raw = ""            # the block as written, given back verbatim when it is not a call
        self.name = ""
        self.emit = True
        self.first_param = True
        self.param: Optional[str] = None
        self.param_str = False
        self.pbuf = ""
        self.pacc = ""           # value text of a non-string parameter, converted when the value ends
        self.pstarted = False
        self.dropped_ws = ""
        self.in_block = False    # inside <tool_call> ... </tool_call> (a bare <function= is not)
        self.call_from_think = False
        if prefix:
            self.buf = prefix

    # ---- output helpers ---------------------------------------------------------------------------------------------
    def _out(self, d: Delta, which: str, s: str) -> None:
        if not s:
            return
        if not self.started[which]:
            s = s.lstrip(" \t\r\n")
            if not s:
                return
            self.started[which] = True
        s = self.ws[which] + s
        body = s.rstrip(" \t\r\n")
        self.ws[which] = s[len(body):]
        if not body:
            return
        if which == "think":
            d.reasoning += body
        else:
            d.content += body
            self.text_seen = True

    def _flush_ws(self, d: Delta, which: str, keep: bool) -> None:
        """Before a marker the held whitespace is dropped; at the end of the reply it is kept."""
        if keep and self.ws[which] and self.started[which]:
            if which == "think":
                d.reasoning += self.ws[which]
            else:
                d.content += self.ws[which]
        self.ws[which] = ""

    def _verbatim(self, d: Delta, s: str) -> None:
        """Give a block that was not a call back to the content exactly as written."""
        if not s:
            return
        if self.started["text"] or s.strip():
            lead = self.ws["text"] if self.started["text"] else ""
            self.ws["text"] = ""
            if not self.started["text"]:
                s = s.lstrip(" \t\r\n")
            self.started["text"] = True
            body = s.rstrip(" \t\r\n")
            self.ws["text"] = s[len(body):]
            d.content += lead + body
            self.text_seen = True

    def _call_id(self) -> str:
        return f"call_{zlib.crc32(f'{self.n_calls}:{self.name}'.encode()) & 0xFFFFFFFF:08x}{self.n_calls:02d}"

    def _start_call(self, d: Delta, name: str) -> None:
        self.name = name
        self.emit = self.max_calls is None or self.n_calls < self.max_calls
        self.index = self.n_calls
        self.n_calls += 1
        self.first_param = True
        self.param = None
        if self.emit:
            d.tool_calls.append({"index": self.index, "id": self._call_id(), "type": "function",
                                 "function": {"name": name, "arguments": ""}})

    def _args(self, d: Delta, piece: str) -> None:
        if self.emit and piece:
            if d.tool_calls and d.tool_calls[-1]["index"] == self.index and "id" not in d.tool_calls[-1]:
                d.tool_calls[-1]["function"]["arguments"] += piece
            else:
                d.tool_calls.append({"index": self.index, "function": {"arguments": piece}})

    def _schema(self, key: str) -> Optional[Dict[str, Any]]:
        fn = self.tools.tools.get(self.name) if self.tools else None
        props = ((fn or {}).get("parameters") or {}).get("properties") or {}
        s = props.get(key)
        return s if isinstance(s, dict) else None

    def _open_param(self, d: Delta, key: str, string_hint: Optional[bool] = None) -> None:
        self.param = key
        sch = self._schema(key)
        t = sch.get("type") if sch else None
        if isinstance(t, list):
            t = next((x for x in t if x != "null"), None)
        # schema types win over the markup's hint; with neither, the value decides when it is complete
        self.param_str = (t == "string") if t is not None else bool(string_hint)
        self.pbuf = ""
        self.pacc = ""
        self.pstarted = False
        self._args(d, ("{" if self.first_param else ", ") + json.dumps(key, ensure_ascii=False) + ": " + ('"' if self.param_str else ""))
        self.first_param = False

    def _param_text(self, d: Delta, s: str, final: bool) -> None:
        """Value text of the open parameter. One newline after the opening tag and one before the closing tag belong
        to the markup, not to the value."""
        if not self.pstarted:
            if not s:
                return
            if s.startswith("\r\n"):
                s = s[2:]
            elif s.startswith("\n"):
                s = s[1:]
            elif s == "\r" and not final:
                self.pbuf = s
                return
            self.pstarted = True
        s = self.pbuf + s
        self.pbuf = ""
        if not final:
            keep = len(s) - len(s.rstrip("\r\n"))           # a trailing newline may be the markup's
            keep = min(keep, 2)
            if keep:
                s, self.pbuf = s[:-keep], s[-keep:]
        else:
            if s.endswith("\r\n"):
                s = s[:-2]
            elif s.endswith("\n"):
                s = s[:-1]
        if self.param_str:
            self._args(d, _jstr(s))
        else:
            self.pacc += s

    def _close_param(self, d: Delta, own_tag: bool = True) -> None:
        if self.param is None:
            return
        self._param_text(d, "", final=True)
        if self.param_str:
            self._args(d, '"')
        else:
            raw, self.pacc = self.pacc, ""
            if not own_tag:
                raw = raw.rstrip()
            v = typed_value(raw, self._schema(self.param))
            self._args(d, json.dumps(v, ensure_ascii=False))
        self.param = None

    def _close_call(self, d: Delta) -> None:
        self._close_param(d, own_tag=False)
        self._args(d, "{}" if self.first_param else "}")
        self.name = ""

    # ---- the state machine ---------------------------------------------------------------------------------------------
    def push(self, text: str) -> Delta:
        d = Delta()
        self.buf += text
        while self._step(d, eof=False):
            pass
        return d

    def finish(self) -> Delta:
        d = Delta()
        while self._step(d, eof=True):
            pass
        for which in ("think", "text"):                 # whitespace that ends the reply is the reply's own
            self._flush_ws(d, which, keep=True)
        return d

    def _take(self, n: int) -> str:
        s, self.buf = self.buf[:n], self.buf[n:]
        return s

    def _step(self, d: Delta, eof: bool) -> bool:
        m = self.mode
        if m in ("think", "text"):
            return self._step_plain(d, eof)
        if m == "preamble":
            return self._step_preamble(d, eof)
        if m == "notcall":
            return self._step_notcall(d, eof)
        if m == "name":
            return self._step_name(d, eof)
        if m == "args":
            return self._step_args(d, eof)
        if m == "between":
            return self._step_between(d, eof)
        if m == "json":
            return self._step_json(d, eof)
        if m == "dsml":
            return self._step_dsml(d, eof)
        if m == "dsml_invoke_name":
            return self._dsml_name(d, eof)
        if m == "dsml_invoke":
            return self._step_dsml_invoke(d, eof)
        raise AssertionError(m)

    def _step_plain(self, d: Delta, eof: bool) -> bool:
        which = self.mode
        if which == "think" and not self.started["think"]:
            # the model opened the block itself although the prompt already had: that tag is not reasoning text
            s = self.buf.lstrip(" \t\r\n")
            if s.startswith(THINK_OPEN):
                self.buf = s[len(THINK_OPEN):]
                return True
            if s and THINK_OPEN.startswith(s) and not eof:
                return False
        markers = [THINK_CLOSE]
        if which == "text" and not self.text_seen:
            markers.append(THINK_OPEN)
        if self.tools_on:
            markers += [DS_CALLS, DS_INVOKE] if self.dsml else [CALL_OPEN]
            if which == "text" and not self.dsml:
                markers.append(FUNC_OPEN)
        pos, tag = _find_first(self.buf, markers)
        if tag is None:
            hold = 0 if eof else _holdback(self.buf, markers)
            self._out(d, which, self._take(len(self.buf) - hold))
            return False
        after = pos + len(tag)
        if tag == THINK_OPEN and (self.text_seen or self.buf[:pos].strip()):
            self._out(d, which, self._take(after))       # a <think> after the content has begun is text
            return True
        if tag == CALL_OPEN and which == "think":
            # the model's own opener is followed by a newline (or is the last thing written); markup quoted in prose is not
            if after >= len(self.buf) and not eof:
                self._out(d, which, self._take(pos))
                return False
            if after < len(self.buf) and self.buf[after] not in "\r\n":
                self._out(d, which, self._take(after))
                return True
        self._out(d, which, self._take(pos))
        self._take(len(tag))
        if tag == THINK_OPEN:
            self.mode = "think"
            self._flush_ws(d, "text", keep=False)
        elif tag == THINK_CLOSE:
            self._flush_ws(d, which, keep=False)
            self.mode = "text"                      # (a stray </think> in content is dropped)
        else:
            # whitespace right before a call is dropped; it is remembered in case the block is no call after all
            self.dropped_ws = self.ws[which] if self.started[which] else ""
            self._flush_ws(d, which, keep=False)
            self.call_from_think = which == "think"
            self.raw = tag
            self.in_block = tag in (CALL_OPEN, DS_CALLS)
            if tag == CALL_OPEN:
                self.mode = "preamble"
            elif tag == FUNC_OPEN:
                self.mode = "name"
            elif tag == DS_CALLS:
                self.mode = "dsml"
            else:
                self.mode = "dsml_invoke_name"
                return self._dsml_name(d, eof)
        return True

    def _not_a_call(self, d: Delta, rest: str = "") -> None:
        """The block was no call: back to the stream it came from, verbatim."""
        text = self.dropped_ws + self.raw + rest
        self.raw = self.dropped_ws = ""
        if self.call_from_think:
            self.mode = "think"
            self._out(d, "think", text)
        else:
            self.mode = "text"
            self._verbatim(d, text)

    def _step_preamble(self, d: Delta, eof: bool) -> bool:
        """Inside <tool_call>, before <function= or a JSON body."""
        s = self.buf.lstrip(" \t\r\n")
        if not s:
            if eof:
                if self.call_from_think:           # cut off right after the opener: the reasoning ends there
                    self.raw = ""
                    self.buf = ""
                    self.mode = "text"
                    return False
                self._not_a_call(d, self._take(len(self.buf)))
            return False
        if s.startswith(FUNC_OPEN):
            self.raw += self._take(len(self.buf) - len(s) + len(FUNC_OPEN))
            self.mode = "name"
            return True
        if FUNC_OPEN.startswith(s) and not eof:
            return False
        if s[0] in "{`":
            self.mode = "json"
            return True
        self.mode = "notcall"
        return True

    def _step_notcall(self, d: Delta, eof: bool) -> bool:
        """Neither a function nor JSON followed the opener: the block is text up to (and including) its closing tag."""
        i = self.buf.find(CALL_CLOSE)
        if i < 0:
            if not eof:
                hold = _holdback(self.buf, [CALL_CLOSE])
                self.raw += self._take(len(self.buf) - hold)
                return False
            self._not_a_call(d, self._take(len(self.buf)))
            return False
        self._not_a_call(d, self._take(i + len(CALL_CLOSE)))
        return True

    def _step_name(self, d: Delta, eof: bool) -> bool:
        i = self.buf.find(">")
        if i < 0:
            if eof:
                name = self._take(len(self.buf)).strip()
                if name:
                    self._start_call(d, name)
                    self._close_call(d)
                self.mode = "text"
            return False
        name = self._take(i + 1)[:-1].strip()
        self.raw += name + ">"
        self._start_call(d, name)
        self.mode = "args"
        return True

    def _step_args(self, d: Delta, eof: bool) -> bool:
        """Inside <function=NAME>: parameters until </function> (or the block's end when that tag is missing)."""
        if self.param is None:
            markers = [PARAM_OPEN, FUNC_CLOSE, CALL_CLOSE, FUNC_OPEN]
            pos, tag = _find_first(self.buf, markers)
            if tag is None:
                if eof:
                    self._take(len(self.buf))
                    self._close_call(d)
                    self.mode = "text"
                    return False
                hold = _holdback(self.buf, markers)
                self._take(len(self.buf) - hold)          # text between parameters is not part of the call
                return False
            self._take(pos)
            if tag == PARAM_OPEN:
                j = self.buf.find(">")
                if j < 0:
                    if eof:
                        self._take(len(self.buf))
                        self._close_call(d)
                        self.mode = "text"
                    return False
                key = self._take(j + 1)[len(PARAM_OPEN):-1].strip()
                self._open_param(d, key)
                return True
            if tag == FUNC_OPEN:                          # the next function started without closing this one
                self._close_call(d)
                self._take(len(FUNC_OPEN))
                self.mode = "name"
                return True
            self._take(len(tag))
            self._close_call(d)
            self.mode = "between" if tag == FUNC_CLOSE and self.in_block else "text"
            return True
        # inside a parameter value
        markers = [PARAM_CLOSE, PARAM_OPEN, FUNC_CLOSE]
        pos, tag = _find_first(self.buf, markers)
        if tag is None:
            hold = 0 if eof else _holdback(self.buf, markers)
            self._param_text(d, self._take(len(self.buf) - hold), final=False)
            if eof:
                self._close_call(d)
                self.mode = "text"
            return False
        self._param_text(d, self._take(pos), final=False)
        if tag == PARAM_CLOSE:
            self._take(len(tag))
            self._close_param(d)
        else:
            self._close_param(d, own_tag=False)           # the closing tag is missing: the next marker ends the value
        return True

    def _step_between(self, d: Delta, eof: bool) -> bool:
        """After </function> inside a block: </tool_call>, another <function= or a new <tool_call> may follow."""
        s = self.buf.lstrip(" \t\r\n")
        markers = [CALL_CLOSE, FUNC_OPEN, CALL_OPEN]
        for t in markers:
            if s.startswith(t):
                self._take(len(self.buf) - len(s) + len(t))
                if t == CALL_CLOSE:
                    self.mode = "text"
                elif t == FUNC_OPEN:
                    self.mode = "name"
                else:
                    self.mode = "preamble"
                    self.raw = CALL_OPEN
                    self.call_from_think = False
                return True
        if not eof and (not s or any(t.startswith(s) for t in markers)):
            return False
        self.mode = "text"
        return bool(self.buf)

    def _step_json(self, d: Delta, eof: bool) -> bool:
        i = self.buf.find(CALL_CLOSE)
        if i < 0 and not eof:
            return False
        body = self._take(i if i >= 0 else len(self.buf))
        closer = self._take(len(CALL_CLOSE)) if i >= 0 else ""
        ok, obj = lenient_json(body)
        if ok and isinstance(obj, dict) and isinstance(obj.get("name"), str):
            args = obj.get("arguments", obj.get("parameters", {}))
            if isinstance(args, str):
                ok2, inner = lenient_json(args)
                args = inner if ok2 and isinstance(inner, dict) else args
            if self.tools and isinstance(args, dict):
                args = self.tools.coerce_arguments(obj["name"], args)
            self._start_call(d, obj["name"])
            self.first_param = False
            self._args(d, args if isinstance(args, str) else json.dumps(args, ensure_ascii=False))
            self.name = ""
            self.raw = ""
            self.mode = "text"
            return True
        self._not_a_call(d, body + closer)
        return True

    # ---- DSML ------------------------------------------------------------------------------------------------------
    def _step_dsml(self, d: Delta, eof: bool) -> bool:
        s = self.buf.lstrip(" \t\r\n")
        for t in (DS_INVOKE, DS_CALLS_END):
            if s.startswith(t):
                self._take(len(self.buf) - len(s) + len(t))
                if t == DS_CALLS_END:
                    self.mode = "text"
                    return True
                self.mode = "dsml_invoke_name"
                return self._dsml_name(d, eof)
        if not eof and (not s or DS_INVOKE.startswith(s) or DS_CALLS_END.startswith(s)):
            return False
        if s:
            self.malformed = True                      # something other than an invoke inside the calls block
        self.mode = "text"
        return bool(self.buf)

    def _dsml_name(self, d: Delta, eof: bool) -> bool:
        i = self.buf.find(">")
        if i < 0:
            if eof:
                self._take(len(self.buf))
                self.mode = "text"
            return False
        head = self._take(i + 1)
        name = head.split('"', 1)[0]
        self._start_call(d, name)
        self.mode = "dsml_invoke"
        return True

    def _step_dsml_invoke(self, d: Delta, eof: bool) -> bool:
        if self.param is None:
            markers = [DS_PARAM, DS_INVOKE_END, DS_INVOKE, DS_CALLS_END]
            pos, tag = _find_first(self.buf, markers)
            if tag is None:
                if eof:
                    self._take(len(self.buf))
                    self._close_call(d)
                    self.mode = "text"
                    return False
                self._take(len(self.buf) - _holdback(self.buf, markers))
                return False
            self._take(pos)
            if tag == DS_PARAM:
                j = self.buf.find(">")
                if j < 0:
                    if eof:
                        self._take(len(self.buf))
                        self._close_call(d)
                        self.mode = "text"
                    return False
                head = self._take(j + 1)[len(DS_PARAM):-1]
                key, _, attrs = head.partition('"')
                self._open_param(d, key, string_hint='string="false"' not in attrs)
                return True
            self._close_call(d)
            if tag == DS_INVOKE_END:
                self._take(len(tag))
                self.mode = "dsml"
            elif tag == DS_INVOKE:                        # the closing tag is missing: the next invoke ends this one
                self.mode = "dsml"
            else:
                self.mode = "dsml"
            return True
        markers = [DS_PARAM_END, DS_PARAM, DS_INVOKE_END]
        pos, tag = _find_first(self.buf, markers)
        if tag is None:
            hold = 0 if eof else _holdback(self.buf, markers)
            self._param_text(d, self._take(len(self.buf) - hold), final=False)
            if eof:
                self._close_call(d)
                self.mode = "text"
            return False
        self._param_text(d, self._take(pos), final=False)
        if tag == DS_PARAM_END:
            self._take(len(tag))
            self._close_param(d)
        else:
            self._close_param(d, own_tag=False)
        return True
