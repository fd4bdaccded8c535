"""API conformance suite: black-box checks of an OpenAI-compatible ferrite_b200 server.

    python -m ferrite_b200.tools.conformance --base-url http://127.0.0.1:8000 [--mock] [--tier quick|heavy|all] [--only NAME]
                                              [--profile hybrid-27b | FILE.json] [--replay DIR]

`--profile` names a model profile (`tools/profiles/*.json`, or a file): the served model's name, its context length, the
least `max_batch_size`, the header that reports the effective sampling, and checks to skip for that model; the `profile`
check compares them with what the server says. `--replay DIR` re-sends the requests a server captured with
`FE_DUMP_REQUESTS=DIR` (`<id>.request.json`): every one must be answered with a well-formed reply, and greedy ones
(temperature 0) twice with the same text.

Every check prints PASS / FAIL; the exit code is 1 on any failure. Tier `quick` (a minute): health and model list, plain
chat (full and streamed, the two must agree), usage accounting, `max_tokens` -> `finish_reason: "length"`, stop strings,
legacy completions, error shapes and limits, streamed chunk framing (`role` first, `[DONE]` last). With `--mock` the
server runs the scripted mock engine, which pins byte for byte: reasoning / answer separation, tool calls in the JSON
and the XML parameter form (full and streamed), arguments checked against the tool's JSON schema, parallel calls, words
before a call, the `tool_choice` forms, escapes and non-ASCII in arguments, a call cut off by `max_tokens`. Tier `heavy`
(scripted long runs): long streamed writes, the loop breaker, the prompt cache across the turns of a conversation,
first byte of a stream while the prompt is still being processed, many requests at once.
Counterpart of the reference's `tools/conformance/run.py` (cases `basic_call`, `generic_schemas`, `parallel_calls`,
`preamble`, `tool_choice`, `special_content`, `cut_off`, `long_write`, `wandering_loop`, `multiturn_cache`, `stopping`,
`liveness_prefill`, `limits`, `reasoning_split`).
"""
from __future__ import annotations

import argparse
import json
import sys
import threading
import time
from typing import Any, Callable, List

from .httpc import Client

TOOLS = [{"type": "function", "function": {
    "name": "get_weather", "description": "weather of a city",
    "parameters": {"type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}},
                   "required": ["city"]}}}]


TOOLS2 = TOOLS + [{"type": "function", "function": {
    "name": "write_file", "description": "write text to a file",
    "parameters": {"type": "object", "properties": {
        "path": {"type": "string"}, "text": {"type": "string"}, "mode": {"type": "string", "enum": ["w", "a"]},
        "lines": {"type": "array", "items": {"type": "integer"}}, "force": {"type": "boolean"}},
        "required": ["path", "text"]}}}]


def validate(v: Any, sc: dict, path: str = "$") -> None:
    """The subset of JSON Schema tool parameters use: type, properties, required, items, enum."""
    t = sc.get("type")
    ok = {"object": isinstance(v, dict), "array": isinstance(v, list), "string": isinstance(v, str),
          "integer": isinstance(v, int) and not isinstance(v, bool), "number": isinstance(v, (int, float)) and not isinstance(v, bool),
          "boolean": isinstance(v, bool), None: True}.get(t, True)
    assert ok, f"{path}: expected {t}, got {type(v).__name__}"
    if "enum" in sc:
        assert v in sc["enum"], f"{path}: {v!r} not in {sc['enum']}"
    if t == "object":
        for k in sc.get("required", []):
            assert k in v, f"{path}: missing {k}"
        for k, x in v.items():
            if k in sc.get("properties", {}):
                validate(x, sc["properties"][k], f"{path}.{k}")
    if t == "array" and "items" in sc:
        for i, x in enumerate(v):
            validate(x, sc["items"], f"{path}[{i}]")


class Suite:
    def __init__(self, client: Client, model: str, mock: bool, tier: str = "quick", only: str = "", profile=None,
                 replay: str = ""):
        self.c, self.model, self.mock, self.tier, self.only = client, model, mock, tier, only
        self.profile, self.replay = profile or {}, replay
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

    def t_profile(self):
        """What the server reports against the model profile."""
        p = self.profile
        _, h = self.c.get("/health")
        if p.get("context"):
            assert int(h.get("max_model_len", 0)) <= int(p["context"]), (h.get("max_model_len"), p["context"])
        if p.get("max_batch_size_min"):
            assert int(h.get("max_batch_size", 0)) >= int(p["max_batch_size_min"]), h
        _, m = self.c.get("/v1/models")
        if p.get("model") and not self.model:
            assert any(d.get("id") == p["model"] for d in m.get("data", [])), (p["model"], m)
        if p.get("effective_sampling_header"):
            _, _, headers = self.c.post("/v1/chat/completions", {"model": self.model, "max_tokens": 4,
                                                                  "messages": [{"role": "user", "content": "hi"}]})
            assert p["effective_sampling_header"] in headers, sorted(headers)

    def t_replay(self):
        """Captured requests, sent again: a well-formed reply each, and the same text twice when greedy."""
        import glob
        import os
        files = sorted(glob.glob(os.path.join(self.replay, "*.request.json")))
        assert files, f"no *.request.json under {self.replay}"
        for f in files:
            with open(f, "r", encoding="utf-8") as fh:
                cap = json.load(fh)
            body = dict(cap["body"], stream=False)
            path = cap.get("meta", {}).get("path") or "/v1/chat/completions"
            texts = []
            for _ in range(2 if float(body.get("temperature", 1) or 0) == 0 else 1):
                status, rep, _ = self.c.post(path, body)
                assert status == 200 and rep.get("choices"), (f, status, str(rep)[:200])
                ch = rep["choices"][0]
                assert ch.get("finish_reason") in ("stop", "length", "tool_calls"), (f, ch.get("finish_reason"))
                msg = ch.get("message") or {}
                texts.append(json.dumps([msg.get("content"), msg.get("tool_calls"), ch.get("text")], sort_keys=True))
                assert rep.get("usage", {}).get("prompt_tokens", 0) > 0, (f, rep.get("usage"))
            assert len(set(texts)) == 1, f"{f}: two greedy replays differ"

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

    def calls_of(self, body) -> list:
        ch = body["choices"][0]
        out = []
        for tc in ch["message"].get("tool_calls") or []:
            assert tc["type"] == "function" and tc["id"], tc
            out.append((tc["function"]["name"], json.loads(tc["function"]["arguments"])))
        return out

    def t_generic_schemas(self):
        args = {"path": "a/b.txt", "text": "x", "mode": "a", "lines": [1, 2, 3], "force": True}
        for kind in ("call", "xcall"):
            b = self.chat(f"[[{kind}:write_file:{json.dumps(args)}]]", tools=TOOLS2, max_tokens=512)
            calls = self.calls_of(b)
            assert len(calls) == 1 and calls[0][0] == "write_file", (kind, calls)
            schema = TOOLS2[1]["function"]["parameters"]
            validate(calls[0][1], schema)                     # typed: the XML form's text values are coerced by the schema
            assert calls[0][1] == args, (kind, calls[0][1])

    def t_parallel_calls(self):
        b = self.chat('[[call:get_weather:{"city": "Oslo"}]][[call:get_weather:{"city": "Rome", "days": 3}]]', tools=TOOLS, max_tokens=512)
        calls = self.calls_of(b)
        assert [c[1].get("city") for c in calls] == ["Oslo", "Rome"], calls
        ids = [tc["id"] for tc in b["choices"][0]["message"]["tool_calls"]]
        assert len(set(ids)) == 2 and b["choices"][0]["finish_reason"] == "tool_calls"

    def t_preamble(self):
        b = self.chat('[[say:Let me check the weather.]][[call:get_weather:{"city": "Oslo"}]]', tools=TOOLS, max_tokens=512)
        m = b["choices"][0]["message"]
        assert (m.get("content") or "").strip() == "Let me check the weather.", m
        assert self.calls_of(b) == [("get_weather", {"city": "Oslo"})]
        assert "<tool_call>" not in (m.get("content") or "")

    def t_tool_choice(self):
        # a named function and "required": the reply is a call whatever the model would have said
        for choice in ({"type": "function", "function": {"name": "get_weather"}}, "required"):
            status, b, _ = self.c.post("/v1/chat/completions", {
                "model": self.model, "messages": [{"role": "user", "content": '[[call:get_weather:{"city": "Oslo"}]]'}],
                "tools": TOOLS, "tool_choice": choice, "max_tokens": 256})
            assert status == 200, (status, b)
            assert b["choices"][0]["finish_reason"] == "tool_calls", (choice, b["choices"][0])
        status, b, _ = self.c.post("/v1/chat/completions", {
            "model": self.model, "messages": [{"role": "user", "content": "x"}], "tools": TOOLS,
            "tool_choice": {"type": "function", "function": {"name": "no_such_tool"}}})
        assert status == 400, (status, b)

    def t_special_content(self):
        text = 'quote " backslash \\ newline\nline two\ttab – ünï©ode 漢字 {"nested": [1, 2]} <b>tag</b>'
        args = {"path": "p", "text": text}
        b = self.chat(f"[[call:write_file:{json.dumps(args, ensure_ascii=False)}]]", tools=TOOLS2, max_tokens=1024)
        assert self.calls_of(b) == [("write_file", args)], self.calls_of(b)
        ev = self.chat_stream(f"[[call:write_file:{json.dumps(args, ensure_ascii=False)}]]", tools=TOOLS2, max_tokens=1024)
        got = "".join(tc.get("function", {}).get("arguments") or "" for e in ev for ch in e["choices"]
                      for tc in ch["delta"].get("tool_calls") or [])
        assert json.loads(got) == args, got

    def t_cut_off(self):
        b = self.chat('[[call:write_file:{"path": "p", "text": "' + "word " * 200 + '"}]]', tools=TOOLS2, max_tokens=40)
        ch = b["choices"][0]
        assert ch["finish_reason"] == "length", ch
        for tc in ch["message"].get("tool_calls") or []:      # whatever is reported must be well formed
            json.loads(tc["function"]["arguments"])

    def t_limits(self):
        post = lambda body: self.c.post("/v1/chat/completions", dict({"model": self.model}, **body))[0]
        assert post({"messages": []}) == 400
        assert post({"messages": [{"role": "user", "content": "x"}], "max_tokens": -1}) == 400
        assert post({"messages": [{"role": "user", "content": "x"}], "temperature": "hot"}) == 400
        assert post({"messages": [{"role": "user", "content": "x"}], "n": 3}) in (200, 400)
        assert post({"messages": [{"role": "wizard", "content": "x"}]}) in (200, 400)
        status, b, _ = self.c.post("/v1/chat/completions", {"model": "no-such-model", "messages": [{"role": "user", "content": "x"}]})
        assert status in (200, 400, 404), (status, b)
        huge = "word " * 20000
        status, b, _ = self.c.post("/v1/chat/completions", {"model": self.model, "messages": [{"role": "user", "content": huge}]})
        assert status in (400, 413), (status, str(b)[:200])
        assert "error" in b

    def t_stopping(self):
        b = self.chat("one two three four five six", stop=["four", "six"])
        c = b["choices"][0]["message"]["content"] or ""
        assert c.rstrip().endswith("three") and b["choices"][0]["finish_reason"] == "stop", b["choices"][0]
        ev = self.chat_stream("one two three four five six", stop=["four"])
        text = "".join(e["choices"][0]["delta"].get("content") or "" for e in ev if e["choices"])
        assert "four" not in text and text.rstrip().endswith("three"), text

    def t_usage_stream(self):
        ev = self.chat_stream("count my tokens", stream_options={"include_usage": True})
        us = [e["usage"] for e in ev if e.get("usage")]
        assert us and us[-1]["total_tokens"] == us[-1]["prompt_tokens"] + us[-1]["completion_tokens"], ev[-2:]

    # ---- heavy tier ---------------------------------------------------------------------------------
    def t_long_write(self):
        n = 200
        ev = self.chat_stream(f"[[repeat:{n}:line of text\n]][[burst:8]]", max_tokens=8000, loop_breaker=False)
        text = "".join(e["choices"][0]["delta"].get("content") or "" for e in ev if e["choices"])
        assert text.count("line of text") == n, text.count("line of text")
        assert any(ch.get("finish_reason") == "stop" for e in ev for ch in e["choices"])

    def t_loop_breaker(self):
        unit = "I will now check the same thing once more to be sure. "
        b = self.chat(f"[[repeat:400:{unit}]][[burst:4]]", max_tokens=8000, loop_breaker=True)
        c = b["choices"][0]["message"]["content"] or ""
        assert 0 < c.count(unit.strip()) < 400, c.count(unit.strip())          # the request ended long before the script did
        assert b["choices"][0]["finish_reason"] in ("stop", "length")

    def t_multiturn_cache(self):
        msgs = [{"role": "user", "content": "remember the number 41 " + "and some padding " * 40}]
        cached = []
        for turn in range(3):
            status, b, _ = self.c.post("/v1/chat/completions", {"model": self.model, "messages": msgs, "max_tokens": 32})
            assert status == 200, b
            cached.append(b["usage"].get("prompt_tokens_details", {}).get("cached_tokens", 0))
            msgs = msgs + [{"role": "assistant", "content": b["choices"][0]["message"]["content"] or ""},
                           {"role": "user", "content": f"turn {turn}: and now?"}]
        assert cached[1] > 0 and cached[2] > cached[1], cached                    # every turn re-uses the turns before it

    def t_liveness_prefill(self):
        t0 = time.time()
        first = None
        for _, e in self.c.stream("/v1/chat/completions", {"model": self.model, "stream": True, "max_tokens": 16,
                                                           "messages": [{"role": "user", "content": "[[slow:1500]]late words"}]}):
            if first is None:
                first = time.time() - t0
        assert first is not None and first < 1.0, first                          # the role chunk does not wait for the prompt

    def t_concurrency(self):
        out, errs = [None] * 8, []

        def one(i):
            try:
                out[i] = self.chat(f"request number {i}", max_tokens=32)["choices"][0]["message"]["content"]
            except Exception as e:  # noqa: BLE001
                errs.append(repr(e))
        ts = [threading.Thread(target=one, args=(i,)) for i in range(8)]
        [t.start() for t in ts]
        [t.join(60) for t in ts]
        assert not errs, errs
        if self.mock:
            assert all(out[i] == f"echo: request number {i}" for i in range(8)), out

    def run(self) -> int:
        quick = [("health", self.t_health), ("models", self.t_models), ("chat full", self.t_chat_full),
                 ("chat stream == full", self.t_chat_stream_matches_full), ("max_tokens -> length", self.t_max_tokens),
                 ("completions", self.t_completions), ("error shape", self.t_bad_request), ("limits", self.t_limits),
                 ("usage in stream", self.t_usage_stream)]
        quick_mock = [("stop string", self.t_stop_string), ("stopping", self.t_stopping),
                      ("reasoning split", self.t_reasoning_split), ("tool call (full)", self.t_tool_call_full),
                      ("tool call (stream)", self.t_tool_call_stream), ("tool_choice none", self.t_tool_choice_none),
                      ("tool_choice forms", self.t_tool_choice), ("generic schemas", self.t_generic_schemas),
                      ("parallel calls", self.t_parallel_calls), ("preamble", self.t_preamble),
                      ("special content", self.t_special_content), ("cut off", self.t_cut_off)]
        heavy = [("concurrency", self.t_concurrency)]
        heavy_mock = [("long write", self.t_long_write), ("loop breaker", self.t_loop_breaker),
                      ("multiturn cache", self.t_multiturn_cache), ("liveness during prefill", self.t_liveness_prefill)]
        todo = []
        if self.tier in ("quick", "all"):
            todo += quick + (quick_mock if self.mock else [])
        if self.tier in ("heavy", "all"):
            todo += ([("models", self.t_models)] if self.tier == "heavy" else []) + heavy + (heavy_mock if self.mock else [])
        if self.profile:
            todo.append(("profile", self.t_profile))
        if self.replay:
            todo.append(("replay", self.t_replay))
        skip = set(self.profile.get("skip", []))
        for name, fn in todo:
            if name in skip:
                continue
            if not self.only or self.only == name or name in ("models",):
                self.check(name, fn)
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
    ap.add_argument("--tier", choices=["quick", "heavy", "all"], default="quick")
    ap.add_argument("--only", default="", help="run one check by name")
    ap.add_argument("--profile", default="", help="model profile: a name under tools/profiles/ or a JSON file")
    ap.add_argument("--replay", default="", help="directory of captured requests (FE_DUMP_REQUESTS) to send again")
    a = ap.parse_args(argv)
    profile = None
    if a.profile:
        import os
        path = a.profile if os.path.exists(a.profile) else os.path.join(os.path.dirname(__file__), "profiles", a.profile + ".json")
        with open(path, "r", encoding="utf-8") as f:
            profile = json.load(f)
    return Suite(Client(a.base_url), a.model, a.mock, a.tier, a.only, profile, a.replay).run()


if __name__ == "__main__":
    sys.exit(main())
