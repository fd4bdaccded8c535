"""Protocol tests through the HTTP app over the mock engine and over the real tiny CPU engine (the shape of the
reference's `crates/fe-server/tests/e2e_mock.rs`, `e2e_batch.rs`, `health_contract.rs`, `utf8_stream.rs`)."""
import asyncio
import json

import pytest
from aiohttp.test_utils import TestClient, TestServer

from ferrite_b200.server.api import ApiError, ChatRequest
from ferrite_b200.server.app import AppState, make_app, snapshot_points
from ferrite_b200.server.engine_api import MockEngine
from ferrite_b200.server.guard import PhaseGuard
from ferrite_b200.server.loopdet import LoopCfg, LoopRule
from ferrite_b200.server.parser import StreamParser, parse_call_body
from ferrite_b200.server.profiles import GenDefaults, resolve_sampling
from ferrite_b200.server.stop import StopMatcher
from ferrite_b200.server.template import ChatTemplate
from ferrite_b200.server.tokenizer import ByteTokenizer, IncrementalDecoder
from ferrite_b200.server.toolcall import ToolSet, coerce

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}}}}]


def run(coro):
    return asyncio.run(coro)


async def client_for(engine_factory, **kw):
    tok = ByteTokenizer(4096)
    app = make_app(lambda: AppState(engine_factory(tok), tok, ChatTemplate(), GenDefaults(), "test-model", **kw))
    c = TestClient(TestServer(app))
    await c.start_server()
    return c


def mock(tok):
    return MockEngine(tok, "test-model", max_batch=4)


async def sse(resp):
    out = []
    async for line in resp.content:
        line = line.decode().strip()
        if line.startswith("data: "):
            out.append(line[6:])
    return out


def chat(content, **kw):
    return {"model": "test-model", "messages": [{"role": "user", "content": content}], **kw}


def test_health_models_and_contract():
    async def go():
        c = await client_for(mock)
        h = await (await c.get("/health")).json()
        assert set(h) >= {"status", "engine", "model", "max_batch_size", "max_model_len", "running", "queued"}
        assert h["status"] == "ok" and h["max_batch_size"] == 4
        m = await (await c.get("/v1/models")).json()
        assert m["data"][0]["id"] == "test-model" and m["data"][0]["context_length"] == 8192
        assert (await c.get("/v1/models/nope")).status == 404
        assert "ferrite_requests_total" in await (await c.get("/metrics")).text()
        await c.close()
    run(go())


def test_reasoning_split_and_stream_equals_non_stream():
    async def go():
        c = await client_for(mock)
        body = chat("hello there [[reason:thinking hard]]", chat_template_kwargs={"enable_thinking": True})
        r = await c.post("/v1/chat/completions", json=body)
        j = await r.json()
        msg = j["choices"][0]["message"]
        assert msg["reasoning_content"].strip() == "thinking hard" and msg["content"] == "echo: hello there"
        assert j["choices"][0]["finish_reason"] == "stop" and j["usage"]["completion_tokens"] > 0
        assert "x-sampling-effective" in r.headers and json.loads(r.headers["x-sampling-effective"])["phase"]
        r = await c.post("/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}})
        chunks = await sse(r)
        assert chunks[-1] == "[DONE]"
        ev = [json.loads(x) for x in chunks[:-1]]
        text = "".join(e["choices"][0]["delta"].get("content", "") for e in ev if e["choices"])
        reason = "".join(e["choices"][0]["delta"].get("reasoning_content", "") for e in ev if e["choices"])
        assert text == msg["content"] and reason.strip() == "thinking hard"
        assert ev[0]["choices"][0]["delta"]["role"] == "assistant"
        assert any(e.get("usage") for e in ev)
        await c.close()
    run(go())


def test_tool_calls_parallel_and_choice():
    async def go():
        c = await client_for(mock)
        body = chat('[[call:get_weather:{"city": "Oslo", "days": "3"}]] [[call:get_weather:{"city": "Rome"}]]', tools=TOOLS)
        j = await (await c.post("/v1/chat/completions", json=body)).json()
        ch = j["choices"][0]
        assert ch["finish_reason"] == "tool_calls" and len(ch["message"]["tool_calls"]) == 2
        a0 = json.loads(ch["message"]["tool_calls"][0]["function"]["arguments"])
        assert a0 == {"city": "Oslo", "days": 3}                       # "3" coerced to the schema's integer
        r = await c.post("/v1/chat/completions", json={**body, "stream": True})
        ev = [json.loads(x) for x in (await sse(r))[:-1]]
        calls = [tc for e in ev for tc in e["choices"][0]["delta"].get("tool_calls", [])]
        # per call: a start delta with id + name, then pieces of the arguments; folded, they are the two calls
        assert sorted(set(tc["index"] for tc in calls)) == [0, 1] and ev[-1]["choices"][0]["finish_reason"] == "tool_calls"
        assert [bool(tc.get("id")) for tc in calls if tc["index"] == 0][0] and sum(1 for tc in calls if tc.get("id")) == 2
        from ferrite_b200.server.parser import merge_tool_calls
        whole = merge_tool_calls(calls)
        assert [json.loads(w["function"]["arguments"]) for w in whole] == [{"city": "Oslo", "days": 3}, {"city": "Rome"}]
        one = await (await c.post("/v1/chat/completions", json={**body, "parallel_tool_calls": False})).json()
        assert len(one["choices"][0]["message"]["tool_calls"]) == 1
        bad = await c.post("/v1/chat/completions", json={**body, "tool_choice": {"type": "function", "function": {"name": "x"}}})
        assert bad.status == 400 and (await bad.json())["error"]["param"] == "tool_choice"
        none = await (await c.post("/v1/chat/completions", json={**chat("plain"), "tools": TOOLS, "tool_choice": "none"})).json()
        assert none["choices"][0]["message"]["content"] == "echo: plain"
        await c.close()
    run(go())


def test_stop_strings_completions_errors_bursts():
    async def go():
        c = await client_for(mock)
        j = await (await c.post("/v1/chat/completions", json=chat("one two three four", stop=["three"]))).json()
        assert j["choices"][0]["message"]["content"] == "echo: one two " and j["choices"][0]["finish_reason"] == "stop"
        j = await (await c.post("/v1/chat/completions", json=chat("abcdefghij [[burst:7]]", max_tokens=9))).json()
        assert j["choices"][0]["finish_reason"] == "length" and j["usage"]["completion_tokens"] == 9
        for bad, status in (({"messages": []}, 400), ({"messages": [{"role": "user", "content": "x"}], "n": 2}, 400),
                            ({"messages": [{"role": "user", "content": "x"}], "temperature": "hot"}, 400)):
            r = await c.post("/v1/chat/completions", json=bad)
            assert r.status == status and "error" in await r.json()
        r = await c.post("/v1/chat/completions", data=b"{not json")
        assert r.status == 400
        j = await (await c.post("/v1/completions", json={"prompt": "<|im_start|>user\nraw text<|im_end|>", "max_tokens": 50})).json()
        assert j["object"] == "text_completion" and j["choices"][0]["text"] == "echo: raw text"
        await c.close()
    run(go())


def test_six_streams_on_four_slots_and_dead_engine():
    async def go():
        c = await client_for(lambda tok: MockEngine(tok, "test-model", max_batch=4, delay_s=0.002))
        rs = await asyncio.gather(*[c.post("/v1/chat/completions", json=chat(f"request number {i}")) for i in range(6)])
        texts = [(await r.json())["choices"][0]["message"]["content"] for r in rs]
        assert texts == [f"echo: request number {i}" for i in range(6)]
        r = await c.post("/v1/chat/completions", json=chat("[[die]]"))
        assert r.status == 500
        h = await c.get("/health")
        assert h.status == 503 and (await h.json())["status"] == "dead"
        assert (await c.post("/v1/chat/completions", json=chat("hi"))).status == 503
        await c.close()
    run(go())


def test_dropped_stream_cancels_the_request_and_frees_its_slot():
    """A client that goes away in the middle of a stream: the request is cancelled, its slot comes back, the next
    request runs (reference `dropped_stream_cancels`, `crates/fe-server/tests/e2e_mock.rs`)."""
    async def go():
        c = await client_for(lambda tok: MockEngine(tok, "test-model", max_batch=1, delay_s=0.01))
        long_reply = "[[repeat:400:word ]]"
        r = await c.post("/v1/chat/completions", json=chat(long_reply, stream=True, max_tokens=4000))
        assert r.status == 200
        got = 0
        async for line in r.content:                        # read a few chunks, then hang up
            if line.startswith(b"data: "):
                got += 1
                if got >= 5:
                    break
        r.close()
        for _ in range(200):                                # the server notices on its next write
            h = await (await c.get("/health")).json()
            if h["running"] == 0 and h["queued"] == 0:
                break
            await asyncio.sleep(0.02)
        assert h["running"] == 0 and h["queued"] == 0, h
        r2 = await c.post("/v1/chat/completions", json=chat("after the drop"))
        assert r2.status == 200 and (await r2.json())["choices"][0]["message"]["content"] == "echo: after the drop"
        await c.close()
    run(go())


def test_watchdog_ends_a_silent_request(monkeypatch):
    monkeypatch.setenv("FE_NO_TOKEN_TIMEOUT", "0.05")
    import ferrite_b200.server.app as appmod
    monkeypatch.setattr(appmod, "KEEPALIVE_S", 0.02)

    async def go():
        c = await client_for(mock)
        r = await c.post("/v1/chat/completions", json=chat("[[silent]]"))
        assert r.status == 500 and "watchdog" in (await r.json())["error"]["message"]
        await c.close()
    run(go())


def test_utf8_never_split_and_stop_holdback():
    tok = ByteTokenizer()
    dec = IncrementalDecoder(tok)
    ids = tok.encode("héllo ✓ 日本")
    out = ""
    for t in ids:
        piece = dec.push([t])
        piece.encode("utf-8")
        assert "�" not in piece
        out += piece
    assert out + dec.flush() == "héllo ✓ 日本"
    sm = StopMatcher(["END"])
    got = ""
    for ch in "abcENxyzEND tail":
        t, hit = sm.push(ch)
        got += t
        if hit:
            break
    assert got == "abcENxyz" and sm.hit == "END"


def test_parser_units():
    ts = ToolSet(TOOLS)
    p = StreamParser(ts, thinking=False)
    text = 'Hi<tool_call><function=get_weather><parameter=city>\nParis\n</parameter><parameter=days>2</parameter></function></tool_call>'
    calls, content = [], ""
    for i in range(0, len(text), 3):
        d = p.push(text[i:i + 3])
        calls += d.tool_calls
        content += d.content
    d = p.finish()
    calls += d.tool_calls
    from ferrite_b200.server.parser import merge_tool_calls
    assert content == "Hi" and json.loads(merge_tool_calls(calls)[0]["function"]["arguments"]) == {"city": "Paris", "days": 2}
    assert parse_call_body('{"name": "f", "arguments": {"a": 1}} trailing', None)["name"] == "f"
    assert parse_call_body("garbage", None) is None
    assert coerce("true", {"type": "boolean"}) is True and coerce("x", {"type": "integer"}) == "x"
    with pytest.raises(ApiError):
        ToolSet([{"type": "function"}])
    with pytest.raises(ApiError):
        ChatRequest.parse({"messages": "no"})


def test_guards_and_profiles_and_snapshots():
    g = PhaseGuard([9, 9], in_thinking=True, max_reasoning=5)
    assert g.feed([1, 2, 3]).force_tokens == [] and g.feed([4, 5]).force_tokens == [9, 9] and not g.in_thinking
    rules = LoopCfg(answer=LoopRule(3, 12))
    g = PhaseGuard([9], in_thinking=False, max_reasoning=None, rules=rules)
    a = g.feed([7, 8] * 12)
    assert a.boost and a.boost_started                               # first sighting: boosted sampling for a while
    assert g.feed([7, 8] * 40).finish is None                       # still inside the boost window
    assert g.feed([7, 8] * 30).finish == "loop"                     # the loop survived the boost: end the reply
    assert g.events.loop_breaks == 2
    from ferrite_b200.server.api import SamplingRequest
    eff = resolve_sampling(SamplingRequest(temperature=0.1), GenDefaults(), thinking=True, ctx_left=100)
    assert eff["temperature"] == 0.1 and eff["top_p"] == 0.95 and eff["max_tokens"] == 100
    tok = ByteTokenizer()
    text = ChatTemplate().render([{"role": "system", "content": "S"}, {"role": "user", "content": "u"},
                                  {"role": "assistant", "content": "a"}, {"role": "user", "content": "v"}])
    pts = snapshot_points(tok, tok.encode(text))
    assert len(pts) == 3 and pts[-1] == len(tok.encode(text))


def test_real_cpu_engine_behind_the_server():
    """Tiny CPU engine + scheduler behind the same HTTP surface: usage accounting, cache hits on a second turn,
    slot release (reference `e2e_batch.rs`)."""
    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.scheduler import Scheduler
    from ferrite_b200.server.engine_api import SchedulerEngine

    def factory(tok):
        cfg = tiny_hybrid()
        eng = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=512, prefill_chunk=64), device="cpu", seed=0)
        return SchedulerEngine(Scheduler(eng), "test-model")

    async def go():
        c = await client_for(factory)
        body = {"messages": [{"role": "system", "content": "You are terse."}, {"role": "user", "content": "hello"}],
                "max_tokens": 8, "temperature": 0}
        j1 = await (await c.post("/v1/chat/completions", json=body)).json()
        assert j1["usage"]["completion_tokens"] <= 8 and j1["usage"]["prompt_tokens"] > 20
        j2 = await (await c.post("/v1/chat/completions", json=body)).json()
        assert j2["choices"][0]["message"] == j1["choices"][0]["message"]          # greedy: same reply
        assert j2["usage"]["prompt_tokens_details"]["cached_tokens"] > 0              # resumed from the snapshot
        h = await (await c.get("/health")).json()
        assert h["running"] == 0 and h["engine"] == "ferrite"
        await c.close()
    run(go())


@pytest.mark.parametrize("kind", ["mtp", "block"])
def test_server_builds_an_engine_with_a_drafter(kind):
    """`--drafter mtp|block`: the server's engine factory taps the target, builds the draft model and hands it to the
    scheduler; greedy replies equal the replies without speculation and drafts were verified."""
    import argparse

    from ferrite_b200.server.__main__ import build_engine
    from ferrite_b200.server.tokenizer import load_tokenizer
    base = dict(model_dir="", preset="tiny", layers=0, weights="bf16", device="cpu", slots=2, prefill_chunk=64,
                max_model_len=256, served_model_name="m", mock=False, engine="ferrite")
    tok = load_tokenizer(None, 4096)
    plain = build_engine(argparse.Namespace(drafter="none", **base), tok)
    spec = build_engine(argparse.Namespace(drafter=kind, **base), tok)
    assert spec.sched.drafter is not None and spec.sched.opts.spec > 0
    import threading

    from ferrite_b200.engine.scheduler import Request, Sampling

    def ask(se, prompt):
        # the server's engine runs its scheduler on a worker thread: submit and wait for the finish event
        out, fin = [], threading.Event()

        def sink(ev):
            if ev.kind == "tokens":
                out.extend(ev.tokens)
            else:
                fin.set()
        se.sched.submit(Request(list(prompt), Sampling(max_tokens=12), sink))
        assert fin.wait(60)
        return out
    p = list(range(5, 45))
    a, b = ask(plain, p), ask(spec, p)
    assert a == b and len(a) == 12 and spec.sched.stats["drafted"] > 0
    plain.sched.stop(); spec.sched.stop()
