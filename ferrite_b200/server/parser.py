"""Streaming reply parser: splits `<think>...</think>` into reasoning, recognises tool calls in the JSON-in-tags form
(`<tool_call>{"name": ..., "arguments": {...}}</tool_call>`) and in the XML parameter form
(`<tool_call><function=NAME><parameter=KEY>value</parameter></function></tool_call>`), and yields OpenAI deltas.
Text that may still turn into a tag is held back, so no tag fragment ever leaks into `content`.
Counterpart of `crates/fe-server/src/parser.rs`."""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .toolcall import ToolSet

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
CALL_OPEN, CALL_CLOSE = "<tool_call>", "</tool_call>"
TAGS = [THINK_OPEN, THINK_CLOSE, CALL_OPEN, CALL_CLOSE]


@dataclass
class Delta:
    reasoning: str = ""
    content: str = ""
    tool_calls: List[Dict[str, Any]] = field(default_factory=list)   # OpenAI tool_call delta objects

    def empty(self) -> bool:
        return not (self.reasoning or self.content or self.tool_calls)


def _held_suffix(buf: str, tags: List[str]) -> int:
    """Length of the longest suffix of buf that is a proper prefix of one of the tags."""
    best = 0
    for t in tags:
        for k in range(min(len(t) - 1, len(buf)), 0, -1):
            if buf.endswith(t[:k]):
                best = max(best, k)
                break
    return best


_FN_RE = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


def parse_call_body(body: str, tools: Optional[ToolSet]) -> Optional[Dict[str, Any]]:
    """Body of one <tool_call>: returns {"name", "arguments" (JSON text)} or None when it cannot be read."""
    b = body.strip()
    m = _FN_RE.search(b)
    if m:
        name = m.group(1)
        args: Dict[str, Any] = {k: v for k, v in _PARAM_RE.findall(m.group(2))}
        if tools:
            args = tools.coerce_arguments(name, args)
        return {"name": name, "arguments": json.dumps(args, ensure_ascii=False)}
    try:
        obj = json.loads(b)
    except json.JSONDecodeError:
        # tolerate a missing closing brace or trailing junk: take the largest prefix that parses
        obj = None
        for end in range(len(b), 0, -1):
            if b[end - 1] != "}":
                continue
            try:
                obj = json.loads(b[:end])
                break
            except json.JSONDecodeError:
                continue
    if not isinstance(obj, dict) or not isinstance(obj.get("name"), str):
        return None
    args = obj.get("arguments", obj.get("parameters", {}))
    if isinstance(args, str):
        try:
            args = json.loads(args)
        except json.JSONDecodeError:
            pass
    if tools:
        args = tools.coerce_arguments(obj["name"], args)
    return {"name": obj["name"], "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}


class StreamParser:
    """Feed text, get deltas. `thinking=True` when the prompt ended inside an open <think> block (the template
    opened it), so the reply starts as reasoning."""

    def __init__(self, tools: Optional[ToolSet] = None, thinking: bool = False, prefix: str = ""):
        self.tools = tools
        self.state = "think" if thinking else "text"
        self.buf = ""
        self.call_buf = ""
        self.n_calls = 0
        self.call_ids: List[str] = []
        self.saw_content = False
        if prefix:
            self.buf = prefix

    def _emit_call(self, d: Delta) -> None:
        call = parse_call_body(self.call_buf, self.tools)
        self.call_buf = ""
        if call is None:
            return
        idx = self.n_calls
        self.n_calls += 1
        cid = f"call_{idx}_{abs(hash(call['name'] + call['arguments'])) % (10 ** 10):010d}"
        self.call_ids.append(cid)
        d.tool_calls.append({"index": idx, "id": cid, "type": "function",
                             "function": {"name": call["name"], "arguments": call["arguments"]}})

    def push(self, text: str) -> Delta:
        d = Delta()
        self.buf += text
        while True:
            if self.state == "call":
                i = self.buf.find(CALL_CLOSE)
                if i < 0:
                    hold = _held_suffix(self.buf, [CALL_CLOSE])
                    self.call_buf += self.buf[:len(self.buf) - hold]
                    self.buf = self.buf[len(self.buf) - hold:]
                    return d
                self.call_buf += self.buf[:i]
                self.buf = self.buf[i + len(CALL_CLOSE):]
                self._emit_call(d)
                self.state = "text"
                continue
            tags = [THINK_CLOSE, THINK_OPEN] if self.state == "think" else [THINK_OPEN, CALL_OPEN]
            pos, tag = -1, None
            for t in tags:
                i = self.buf.find(t)
                if i >= 0 and (pos < 0 or i < pos):
                    pos, tag = i, t
            if tag is None:
                hold = _held_suffix(self.buf, tags)
                out, self.buf = self.buf[:len(self.buf) - hold], self.buf[len(self.buf) - hold:]
                self._text(d, out)
                return d
            self._text(d, self.buf[:pos])
            self.buf = self.buf[pos + len(tag):]
            if tag == THINK_OPEN:
                self.state = "think"
            elif tag == THINK_CLOSE:
                self.state = "text"
                self.buf = self.buf.lstrip("\n") if not self.saw_content else self.buf
            elif tag == CALL_OPEN:
                self.state = "call"

    def _text(self, d: Delta, s: str) -> None:
        if not s:
            return
        if self.state == "think":
            d.reasoning += s
        else:
            if not self.saw_content:
                s = s.lstrip("\n")
                if not s:
                    return
            self.saw_content = True
            d.content += s

    def finish(self) -> Delta:
        """End of stream: flush held text; an unterminated call is parsed as far as it goes."""
        d = Delta()
        if self.state == "call":
            self.call_buf += self.buf
            self.buf = ""
            self._emit_call(d)
        else:
            self._text(d, self.buf)
            self.buf = ""
        return d
