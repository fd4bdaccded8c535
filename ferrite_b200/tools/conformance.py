"""API conformance suite: black-box checks of an OpenAI-compatible ferrite_b200 server.

    python -m ferrite_b200.tools.conformance --base-url http://127.0.0.1:8000 [--mock]

Checks (each prints PASS/FAIL; exit code 1 on any failure): health and model list, plain chat (full and streamed, the
two must agree), usage accounting, `max_tokens` -> `finish_reason: "length"`, stop strings, legacy completions, error
shape for bad requests, streamed chunk framing (`role` first, `[DONE]` last). With `--mock` the server runs the scripted
mock engine, which lets the suite also pin reasoning/answer separation and tool calls (full and streamed, JSON
arguments, `finish_reason: "tool_calls"`) byte for byte. Counterpart of the reference's `tools/conformance/run.py`.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Callable, List

from .httpc import Client

TOOLS = [{"type": "function", "function": {
    "name": "get_weather", "description": "weather of a city",
    "parameters": {"type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}},
                   "required": ["city"]}}}]


class Suite:
    def __init__(self, client: Client, model: str, mock: bool):
        self.c, self.model, self.mock = client, model, mock
        self.results: List[tuple] = []

    def check(self, name: str, fn: Callable[[], None]) -> None:
        try:
            fn()
            self.results.append((name, True, ""))
        except Exception as e:  # noqa: BLE001 - a failed check must not stop the suite
            self.results.append((name, False, f"{type(e).__name__}: {e}"))

    def chat(self, content: str, **kw):
        status, body, _ = self.c.post("/v1/chat/completions", dict(
            {"model": self.model, "messages": [{"role": "user", "content": content}], "max_tokens": 64}, **kw))
        assert status == 200, (status, body)
        return body

    def chat_stream(self, content: str, **kw):
        events = [e for _, e in self.c.stream("/v1/chat/completions", dict(
            {"model": self.model, "messages": [{"role": "user", "content": content}], "max_tokens": 64}, **kw))]
        assert events and events[-1] is None, "stream did not end with [DONE]"
        return events[:-1]

    # ---- checks -------------------------------------------------------------------------------------
    def t_health(self):
        status, body = self.c.get("/health")
        assert status == 200 and body.get("status") == "ok", (status, body)

    def t_models(self):
        status, body = self.c.get("/v1/models")
        assert status == 200 and body["object"] == "list" and body["data"], body
        if not self.model:
            self.model = body["data"][0]["id"]
        assert any(m["id"] == self.model for m in body["data"])

    def t_chat_full(self):
        b = self.chat("say hello")
        ch = b["choices"][0]
        assert b["object"] == "chat.completion" and ch["message"]["role"] == "assistant"
        assert ch["finish_reason"] in ("stop", "length")
        u = b["usage"]
        assert u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"] and u["prompt_tokens"] > 0

    def t_chat_stream_matches_full(self):
        full = self.chat("stream check", temperature=0)
        ev = self.chat_stream("stream check", temperature=0)
        assert ev[0]["choices"][0]["delta"].get("role") == "assistant", ev[0]
        text = "".join(e["choices"][0]["delta"].get("content") or "" for e in ev if e["choices"])
        assert text == (full["choices"][0]["message"]["content"] or ""), (text, full)
        assert any(e["choices"] and e["choices"][0].get("finish_reason") for e in ev)

    def t_max_tokens(self):
        b = self.chat("please write a very long answer about nothing in particular, thank you", max_tokens=3)
        assert b["usage"]["completion_tokens"] <= 3
        assert b["choices"][0]["finish_reason"] == "length", b["choices"][0]

    def t_completions(self):
        status, b, _ = self.c.post("/v1/completions", {"model": self.model, "prompt": "abc", "max_tokens": 8})
        assert status == 200 and b["object"] == "text_completion" and "text" in b["choices"][0], b

    def t_bad_request(self):
        status, b, _ = self.c.post("/v1/chat/completions", {"model": self.model, "messages": "nope"})
        assert status == 400 and "error" in b and "message" in b["error"], (status, b)

    def t_stop_string(self):
        b = self.chat("alpha beta gamma delta", stop=["gamma"])
        assert "gamma" not in (b["choices"][0]["message"]["content"] or ""), b
        assert b["choices"][0]["finish_reason"] == "stop"

    # mock-only (scripted) checks
    def t_reasoning_split(self):
        b = self.chat("[[reason:think a little]]the answer")
        m = b["choices"][0]["message"]
        assert (m.get("reasoning_content") or "").strip() == "think a little", m
        assert m["content"].strip() == "echo: the answer", m

    def t_tool_call_full(self):
        b = self.chat('[[call:get_weather:{"city": "Oslo", "days": 2}]]', tools=TOOLS, max_tokens=512)
        ch = b["choices"][0]
        assert ch["finish_reason"] == "tool_calls", ch
        tc = ch["message"]["tool_calls"][0]
        assert tc["type"] == "function" and tc["function"]["name"] == "get_weather"
        assert json.loads(tc["function"]["arguments"]) == {"city": "Oslo", "days": 2}

    def t_tool_call_stream(self):
        ev = self.chat_stream('[[call:get_weather:{"city": "Oslo"}]]', tools=TOOLS, max_tokens=512)
        name, args = "", ""
        for e in ev:
            for ch in e["choices"]:
                for tc in ch["delta"].get("tool_calls") or []:
                    name += tc.get("function", {}).get("name") or ""
                    args += tc.get("function", {}).get("arguments") or ""
        assert name == "get_weather" and json.loads(args) == {"city": "Oslo"}, (name, args)
        assert any(ch.get("finish_reason") == "tool_calls" for e in ev for ch in e["choices"])

    def t_tool_choice_none(self):
        b = self.chat("plain words", tools=TOOLS, tool_choice="none")
        assert not b["choices"][0]["message"].get("tool_calls"), b

    def run(self) -> int:
        self.check("health", self.t_health)
        self.check("models", self.t_models)
        self.check("chat full", self.t_chat_full)
        self.check("chat stream == full", self.t_chat_stream_matches_full)
        self.check("max_tokens -> length", self.t_max_tokens)
        self.check("completions", self.t_completions)
        self.check("error shape", self.t_bad_request)
        if self.mock:
            self.check("stop string", self.t_stop_string)
            self.check("reasoning split", self.t_reasoning_split)
            self.check("tool call (full)", self.t_tool_call_full)
            self.check("tool call (stream)", self.t_tool_call_stream)
            self.check("tool_choice none", self.t_tool_choice_none)
        bad = 0
        for name, ok, msg in self.results:
            print(("PASS " if ok else "FAIL ") + name + ("" if ok else "  -- " + msg))
            bad += 0 if ok else 1
        print(f"{len(self.results) - bad}/{len(self.results)} checks passed")
        return 1 if bad else 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="")
    ap.add_argument("--mock", action="store_true", help="the server runs the scripted mock engine")
    a = ap.parse_args(argv)
    return Suite(Client(a.base_url), a.model, a.mock).run()


if __name__ == "__main__":
    sys.exit(main())
