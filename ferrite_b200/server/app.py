"""OpenAI-compatible HTTP server: `/health`, `/v1/health`, `/v1/models`, `/v1/models/{id}`, `/v1/chat/completions`,
`/v1/completions`, `/metrics`; SSE streaming with reasoning and tool-call deltas, usage and llama-server-style
timings, stop strings, tool_choice enforcement, sampling profiles with the `x-sampling-effective` header, a watchdog
(no-token timeout, wall limit), keep-alive pings, request capture for replay, and a 503 health once the engine died.

Counterpart of `crates/fe-server/src/server.rs` (`router` `:305`, `health` `:322-340`, `resolve_sampling` `:467`,
`prepare_chat` `:580`, `Pipeline` `:857`, `Driver` `:978`, `stream_response` `:1275`, `full_response` `:1338`).
The engine side is token-level (`engine_api.EngineBase`); everything textual happens here.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
import uuid
from typing import Any, Dict, List, Optional, Tuple

from aiohttp import web

from ..engine.sampler import Sampling
from .api import ApiError, ChatRequest, CompletionRequest
from .engine_api import EngineBase, GenEvent, GenRequest
from .guard import PhaseGuard
from .loopdet import LoopCfg
from .parser import Delta, StreamParser, merge_tool_calls
from .profiles import GenDefaults, resolve_sampling
from .stop import StopMatcher
from .template import ChatTemplate
from .tokenizer import IncrementalDecoder
from .toolcall import ToolSet

BODY_LIMIT = 32 << 20
KEEPALIVE_S = 10.0


def snapshot_points(tok, ids: List[int]) -> List[int]:
    """Prompt positions worth a state snapshot: the end of the system message and the start of every assistant
    turn (reference `Marks::points`, `crates/fe-server/src/snapshots.rs:39`)."""
    marks: List[int] = []
    try:
        start = tok.encode("<|im_start|>assistant\n")
        end = tok.encode("<|im_end|>\n")
    except Exception:
        return marks
    n = len(ids)
    first_end = None
    for i in range(n - len(end) + 1):
        if ids[i:i + len(end)] == end:
            first_end = i + len(end)
            break
    if first_end:
        marks.append(first_end)
    for i in range(n - len(start) + 1):
        if ids[i:i + len(start)] == start:
            marks.append(i + len(start))
    return sorted(set(m for m in marks if 0 < m <= n))


class Pipeline:
    """ids -> UTF-8-safe text -> stop strings -> reasoning / content / tool-call deltas (reference `Pipeline`)."""

    def __init__(self, tok, stops: List[str], include_stop: bool, tools: Optional[ToolSet], thinking: bool, prefix: str = "",
                 raw: bool = False, max_tool_calls: Optional[int] = None, dsml: bool = False):
        self.dec = IncrementalDecoder(tok)
        self.stop = StopMatcher(stops, include_stop)
        self.parser = None if raw else StreamParser(tools, thinking, prefix, max_tool_calls=max_tool_calls, dsml=dsml)
        self.stopped = False
        self.text = ""

    def push(self, ids: List[int]) -> Delta:
        if self.stopped:
            return Delta()
        text, hit = self.stop.push(self.dec.push(ids))
        self.stopped = hit
        self.text += text
        return self.parser.push(text) if self.parser else Delta(content=text)

    def finish(self) -> Delta:
        tail = ""
        if not self.stopped:
            tail = self.stop.push(self.dec.flush())[0] + self.stop.flush()
        self.text += tail
        if self.parser is None:
            return Delta(content=tail)
        d = self.parser.push(tail) if tail else Delta()
        f = self.parser.finish()
        d.reasoning += f.reasoning
        d.content += f.content
        d.tool_calls += f.tool_calls
        return d


class AppState:
    def __init__(self, engine: EngineBase, tok, template: ChatTemplate, defaults: GenDefaults, served_name: str,
                 max_concurrent: int = 16, capture_dir: Optional[str] = None):
        self.engine, self.tok, self.template, self.defaults = engine, tok, template, defaults
        self.served_name = served_name
        self.sem = asyncio.Semaphore(max_concurrent)
        self.capture_dir = capture_dir or os.environ.get("FE_DUMP_REQUESTS")
        self.started = time.time()
        self.counters = {"requests": 0, "completion_tokens": 0, "prompt_tokens": 0, "cached_tokens": 0, "errors": 0}
        self.no_token_timeout = float(os.environ.get("FE_NO_TOKEN_TIMEOUT", defaults.no_token_timeout_s))
        self.wall_limit = float(os.environ.get("FE_REPLY_WALL_LIMIT", defaults.reply_wall_limit_s))


def _err(e: ApiError) -> web.Response:
    return web.json_response(e.body(), status=e.status)


async def health(request: web.Request) -> web.Response:
    st: AppState = request.app[STATE]
    info = st.engine.info()
    dead = st.engine.dead()
    load = st.engine.load()
    body = {"status": "ok" if not dead else "dead", "engine": info.name, "model": st.served_name,
            "max_batch_size": info.max_batch_size, "max_model_len": info.max_model_len,
            "running": load["running"], "queued": load["queued"]}
    if dead:
        body["error"] = dead
    return web.json_response(body, status=503 if dead else 200)


async def models(request: web.Request) -> web.Response:
    st: AppState = request.app[STATE]
    info = st.engine.info()
    card = {"id": st.served_name, "object": "model", "created": int(st.started), "owned_by": "ferrite",
            "context_length": info.max_model_len, "max_model_len": info.max_model_len}
    mid = request.match_info.get("id")
    if mid is not None:
        if mid != st.served_name:
            return _err(ApiError(404, f"model {mid!r} not found", "not_found_error", code="model_not_found"))
        return web.json_response(card)
    return web.json_response({"object": "list", "data": [card]})


async def metrics(request: web.Request) -> web.Response:
    st: AppState = request.app[STATE]
    load = st.engine.load()
    lines = [f"ferrite_{k}_total {v}" for k, v in st.counters.items()]
    lines += [f"ferrite_running {load['running']}", f"ferrite_queued {load['queued']}",
              f"ferrite_uptime_seconds {time.time() - st.started:.1f}"]
    lines += [f"ferrite_engine_{k} {v}" for k, v in st.engine.metrics().items()]
    return web.Response(text="\n".join(lines) + "\n", content_type="text/plain")


STATE: "web.AppKey[AppState]" = web.AppKey("state", AppState)


def _capture(st: AppState, kind: str, body: Any, meta: Dict[str, Any]) -> None:
    if not st.capture_dir:
        return
    os.makedirs(st.capture_dir, exist_ok=True)
    rid = meta["id"]
    with open(os.path.join(st.capture_dir, f"{rid}.{kind}.json"), "w") as f:
        json.dump({"body": body, "meta": meta}, f)


class Prepared:
    def __init__(self):
        self.ids: List[int] = []
        self.sampling: Sampling = Sampling()
        self.effective: Dict[str, Any] = {}
        self.tools: Optional[ToolSet] = None
        self.thinking = False
        self.prefix = ""
        self.stops: List[str] = []
        self.include_stop = False
        self.snapshots: List[int] = []
        self.guard: Optional[PhaseGuard] = None
        self.raw = False
        self.max_tool_calls: Optional[int] = None     # parallel_tool_calls: false -> 1
        self.dsml = False                             # the template writes DSML tool calls


def prepare_chat(st: AppState, req: ChatRequest) -> Prepared:
    p = Prepared()
    tools = ToolSet(req.tools) if req.tool_choice != "none" else ToolSet([])
    p.dsml = "DSML" in getattr(st.template, "source", "")
    p.max_tool_calls = None if req.parallel_tool_calls else 1
    forced = tools.resolve_choice(req.tool_choice, p.dsml)
    think = req.enable_thinking
    kwargs = {} if think is None else {"enable_thinking": bool(think)}
    text = st.template.render(req.messages, [dict(t) for t in req.tools] if tools else None, True, **kwargs)
    p.thinking = text.rstrip().endswith("<think>") or (think is True and not text.rstrip().endswith("</think>"))
    if forced is not None:
        if p.thinking:                      # a forced call skips reasoning
            text += "\n</think>\n\n" if text.rstrip().endswith("<think>") else ""
            p.thinking = False
        text += forced.opener
        p.prefix = forced.opener
    p.ids = st.tok.encode(text)
    info = st.engine.info()
    if len(p.ids) >= info.max_model_len:
        raise ApiError(400, f"prompt of {len(p.ids)} tokens exceeds the context of {info.max_model_len}",
                       code="context_length_exceeded")
    eff = resolve_sampling(req.sampling, st.defaults, p.thinking, info.max_model_len - len(p.ids))
    p.effective = eff
    stop_ids = list(req.sampling.stop_token_ids)
    if not req.sampling.ignore_eos:
        stop_ids += list(st.tok.eos_ids)
    p.sampling = Sampling(temperature=eff["temperature"], top_k=eff["top_k"], top_p=eff["top_p"], min_p=eff["min_p"],
                          presence_penalty=eff["presence_penalty"], frequency_penalty=eff["frequency_penalty"],
                          repetition_penalty=eff["repetition_penalty"], seed=eff["seed"], max_tokens=eff["max_tokens"],
                          stop_ids=stop_ids, banned_first=list(st.tok.eos_ids))
    p.tools = tools
    p.stops, p.include_stop = req.sampling.stop, req.sampling.include_stop_str_in_output
    p.snapshots = snapshot_points(st.tok, p.ids)
    max_r = req.max_reasoning_tokens if req.max_reasoning_tokens is not None else st.defaults.max_reasoning_tokens
    lb = st.defaults.loop_breaker if req.loop_breaker is None else bool(req.loop_breaker)
    p.guard = PhaseGuard(st.tok.encode("</think>"), p.thinking, max_r, lb, LoopCfg.from_json(getattr(st.defaults, "loop_rules", None)),
                         close_ids=st.tok.encode("\n</think>\n\n"),
                         call_marks=[st.tok.encode(m) for m in ("<tool_call>", "<function=")] if tools else (),
                         detok=lambda ids: st.tok.decode(list(ids)))
    return p


def prepare_completion(st: AppState, req: CompletionRequest) -> Prepared:
    p = Prepared()
    p.raw = True
    p.ids = st.tok.encode(req.prompt) if isinstance(req.prompt, str) else [int(x) for x in req.prompt]
    info = st.engine.info()
    if not p.ids:
        raise ApiError(400, "empty prompt", param="prompt")
    if len(p.ids) >= info.max_model_len:
        raise ApiError(400, "prompt exceeds the context length", code="context_length_exceeded")
    eff = resolve_sampling(req.sampling, st.defaults, False, info.max_model_len - len(p.ids))
    p.effective = eff
    stop_ids = list(req.sampling.stop_token_ids) + ([] if req.sampling.ignore_eos else list(st.tok.eos_ids))
    p.sampling = Sampling(temperature=eff["temperature"], top_k=eff["top_k"], top_p=eff["top_p"], min_p=eff["min_p"],
                          presence_penalty=eff["presence_penalty"], frequency_penalty=eff["frequency_penalty"],
                          repetition_penalty=eff["repetition_penalty"], seed=eff["seed"], max_tokens=eff["max_tokens"],
                          stop_ids=stop_ids)
    p.stops, p.include_stop = req.sampling.stop, req.sampling.include_stop_str_in_output
    return p


class Driver:
    """Per-request task: receives engine events, runs the pipeline, enforces the watchdog (reference `Driver`)."""

    def __init__(self, st: AppState, p: Prepared):
        self.st, self.p = st, p
        self.q: "asyncio.Queue[GenEvent]" = asyncio.Queue()
        self.loop = asyncio.get_running_loop()
        self.pipe = Pipeline(st.tok, p.stops, p.include_stop, p.tools, p.thinking, p.prefix, raw=p.raw,
                             max_tool_calls=p.max_tool_calls, dsml=p.dsml)
        self.req = GenRequest(p.ids, p.sampling, p.snapshots)
        self.completion_tokens = 0
        self.finish_reason = "stop"
        self.timings: Dict[str, float] = {}
        self.error: Optional[str] = None
        self.forced_tokens: List[int] = []
        if p.guard is not None:
            self.req.guard = self._guard

    def _guard(self, toks: List[int]):
        act = self.p.guard.feed(toks, "")
        s = self.req.sampling
        if act.boost_started:
            # a loop in the answer: sample the next stretch with the recovery values (a greedy request leaves its cycle)
            self._own_sampling = (s.temperature, s.top_p)
            rules = self.p.guard.tracker.rules
            s.temperature, s.top_p = max(s.temperature, rules.recover_temperature), min(s.top_p, rules.recover_top_p)
        elif act.boost_ended and getattr(self, "_own_sampling", None):
            s.temperature, s.top_p = self._own_sampling
            self._own_sampling = None
        if act.finish:
            return act.finish
        return act.force_tokens or None

    def start(self) -> None:
        def sink(ev: GenEvent):
            self.loop.call_soon_threadsafe(self.q.put_nowait, ev)
        self.st.engine.submit(self.req, sink)

    async def deltas(self):
        """Async iterator of Delta objects; ends after the finish event. Raises ApiError on engine errors."""
        t_start = time.time()
        last = time.time()
        while True:
            timeout = KEEPALIVE_S
            try:
                ev = await asyncio.wait_for(self.q.get(), timeout)
            except asyncio.TimeoutError:
                now = time.time()
                if self.st.no_token_timeout and now - last > self.st.no_token_timeout:
                    self.req.cancel.set()
                    self.finish_reason, self.error = "error", "no token from the engine within the watchdog limit"
                    return
                if self.st.wall_limit and now - t_start > self.st.wall_limit:
                    self.req.cancel.set()
                    self.finish_reason = "length"
                    return
                yield None                       # keep-alive tick
                continue
            last = time.time()
            if ev.kind == "tokens":
                self.completion_tokens += len(ev.tokens)
                d = self.pipe.push(ev.tokens)
                if not d.empty():
                    yield d
                if self.pipe.stopped:
                    self.req.cancel.set()
                    self.finish_reason = "stop"
            elif ev.kind == "finish":
                if not self.pipe.stopped:
                    self.finish_reason = {"stop": "stop", "length": "length", "cancelled": "stop", "guard": "stop",
                                          "loop": "stop"}.get(ev.reason, ev.reason or "stop")
                self.timings = ev.timings
                d = self.pipe.finish()
                if not d.empty():
                    yield d
                if self.pipe.parser is not None and self.pipe.parser.n_calls > 0:
                    self.finish_reason = "tool_calls"
                return
            else:
                self.error = ev.message or "engine error"
                self.finish_reason = "error"
                return

    def usage(self) -> Dict[str, Any]:
        cached = int(self.timings.get("cache_n", 0))
        return {"prompt_tokens": len(self.p.ids), "completion_tokens": self.completion_tokens,
                "total_tokens": len(self.p.ids) + self.completion_tokens,
                "prompt_tokens_details": {"cached_tokens": cached}}


def _sse(obj: Any) -> bytes:
    return ("data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n").encode("utf-8")


async def _run(request: web.Request, chat: bool) -> web.StreamResponse:
    st: AppState = request.app[STATE]
    st.engine.incoming(+1)              # until the request is handed to the engine (or refused)
    counted = [True]

    def handed_over():
        if counted[0]:
            counted[0] = False
            st.engine.incoming(-1)
    try:
        raw = await request.read()
        if len(raw) > BODY_LIMIT:
            raise ApiError(413, "request body too large")
        try:
            body = json.loads(raw)
        except json.JSONDecodeError as e:
            raise ApiError(400, f"invalid JSON: {e}")
        if st.engine.dead():
            raise ApiError(503, "engine is not running", "server_error")
        if chat:
            req = ChatRequest.parse(body)
            prep = prepare_chat(st, req)
        else:
            req = CompletionRequest.parse(body)
            prep = prepare_completion(st, req)
    except ApiError as e:
        handed_over()
        st.counters["errors"] += 1
        return _err(e)
    except BaseException:
        handed_over()
        raise
    rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
    created = int(time.time())
    _capture(st, "request", body, {"id": rid, "path": request.path, "prompt_tokens": len(prep.ids)})
    st.counters["requests"] += 1
    headers = {"x-sampling-effective": json.dumps(prep.effective, ensure_ascii=False)}
    obj = "chat.completion" if chat else "text_completion"
    try:
        await st.sem.acquire()
    except BaseException:
        handed_over()
        raise
    try:
        drv = Driver(st, prep)
        drv.start()
        handed_over()
        return await _respond(st, request, req, prep, drv, rid, created, headers, obj, chat)
    finally:
        handed_over()
        st.sem.release()


async def _respond(st, request, req, prep, drv, rid, created, headers, obj, chat):
    if True:
        if req.stream:
            resp = web.StreamResponse(status=200, headers={**headers, "Content-Type": "text/event-stream; charset=utf-8",
                                                           "Cache-Control": "no-cache"})
            await resp.prepare(request)
            base = {"id": rid, "object": obj + ".chunk" if chat else obj, "created": created, "model": st.served_name}
            try:
                if chat:
                    await resp.write(_sse({**base, "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""},
                                                                "finish_reason": None}]}))
                async for d in drv.deltas():
                    if d is None:
                        await resp.write(b": keep-alive\n\n")
                        continue
                    if chat:
                        delta: Dict[str, Any] = {}
                        if d.reasoning:
                            delta["reasoning_content"] = d.reasoning
                        if d.content:
                            delta["content"] = d.content
                        if d.tool_calls:
                            delta["tool_calls"] = d.tool_calls
                        await resp.write(_sse({**base, "choices": [{"index": 0, "delta": delta, "finish_reason": None}]}))
                    elif d.content:
                        await resp.write(_sse({**base, "choices": [{"index": 0, "text": d.content, "finish_reason": None}]}))
                if drv.error:
                    await resp.write(_sse({"error": {"message": drv.error, "type": "server_error", "param": None, "code": None}}))
                else:
                    fin = {"index": 0, "finish_reason": drv.finish_reason}
                    fin.update({"delta": {}} if chat else {"text": ""})
                    last = {**base, "choices": [fin]}
                    if drv.timings:
                        last["timings"] = drv.timings
                    await resp.write(_sse(last))
                    if req.include_usage:
                        await resp.write(_sse({**base, "choices": [], "usage": drv.usage()}))
                await resp.write(_sse("[DONE]"))
            except (ConnectionResetError, asyncio.CancelledError):
                drv.req.cancel.set()               # client went away: free the slot
                raise
            finally:
                drv.req.cancel.set() if drv.finish_reason == "error" else None
                _account(st, drv)
            return resp
        reasoning, content, calls = "", "", []
        async for d in drv.deltas():
            if d is None:
                continue
            reasoning += d.reasoning
            content += d.content
            calls += d.tool_calls
        _account(st, drv)
        if drv.error:
            return _err(ApiError(500, drv.error, "server_error"))
        if chat:
            msg: Dict[str, Any] = {"role": "assistant", "content": content if (content or not calls) else None}
            if reasoning:
                msg["reasoning_content"] = reasoning
            if calls:
                # streamed pieces (name first, then argument text) fold into whole calls
                msg["tool_calls"] = [{k: v for k, v in c.items() if k != "index"} for c in merge_tool_calls(calls)]
            choice = {"index": 0, "message": msg, "finish_reason": drv.finish_reason}
        else:
            choice = {"index": 0, "text": content, "finish_reason": drv.finish_reason, "logprobs": None}
        out = {"id": rid, "object": obj, "created": created, "model": st.served_name, "choices": [choice],
               "usage": drv.usage()}
        if drv.timings:
            out["timings"] = drv.timings
        return web.json_response(out, headers=headers, dumps=lambda o: json.dumps(o, ensure_ascii=False))


def _account(st: AppState, drv: Driver) -> None:
    st.counters["completion_tokens"] += drv.completion_tokens
    st.counters["prompt_tokens"] += len(drv.p.ids)
    st.counters["cached_tokens"] += int(drv.timings.get("cache_n", 0))
    if drv.error:
        st.counters["errors"] += 1


async def chat_completions(request: web.Request) -> web.StreamResponse:
    return await _run(request, True)


async def completions(request: web.Request) -> web.StreamResponse:
    return await _run(request, False)


def make_app(state_factory) -> web.Application:
    """state_factory() -> AppState is called inside the running loop (it creates asyncio primitives)."""
    app = web.Application(client_max_size=BODY_LIMIT + 1024)

    async def on_start(app):
        app[STATE] = state_factory()

    async def on_stop(app):
        app[STATE].engine.shutdown()

    app.on_startup.append(on_start)
    app.on_cleanup.append(on_stop)
    app.router.add_get("/health", health)
    app.router.add_get("/v1/health", health)
    app.router.add_get("/v1/models", models)
    app.router.add_get("/v1/models/{id}", models)
    app.router.add_get("/metrics", metrics)
    app.router.add_post("/v1/chat/completions", chat_completions)
    app.router.add_post("/v1/completions", completions)
    return app
