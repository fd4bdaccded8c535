"""Token-level boundary between the protocol layer and an engine: ids in, ids out.
Counterpart of `crates/fe-server/src/engine.rs` (`SamplingParams`, `CancelToken`, `GenRequest`, `FinishReason`,
`Timings`, `GenEvent`, `TokenSink`, `EngineInfo`, trait `Engine`) and of the adapters `ferrite.rs` / `mock.rs`."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from ..engine.sampler import Sampling


@dataclass
class EngineInfo:
    name: str
    model: str
    max_batch_size: int
    max_model_len: int
    vocab_size: int


@dataclass
class GenRequest:
    ids: List[int]
    sampling: Sampling
    snapshots: List[int] = field(default_factory=list)
    cancel: threading.Event = field(default_factory=threading.Event)
    guard: Optional[Callable[[List[int]], Optional[str]]] = None


@dataclass
class GenEvent:
    kind: str                                  # "tokens" | "finish" | "error"
    tokens: List[int] = field(default_factory=list)
    reason: str = ""
    timings: Dict[str, float] = field(default_factory=dict)
    message: str = ""


TokenSink = Callable[[GenEvent], None]


class EngineBase:
    def info(self) -> EngineInfo:
        raise NotImplementedError

    def submit(self, req: GenRequest, sink: TokenSink) -> None:
        raise NotImplementedError

    def dead(self) -> Optional[str]:
        return None

    def load(self) -> Dict[str, int]:
        return {"running": 0, "queued": 0}

    def metrics(self) -> Dict[str, float]:
        return {}

    def incoming(self, delta: int) -> None:
        """The server is preparing (+1) / has handed over or dropped (-1) a request: an idle engine that has just been
        woken waits a little for requests that are still being tokenised (reference `Engine::incoming`)."""

    def shutdown(self) -> None:
        pass


class SchedulerEngine(EngineBase):
    """Adapter over `engine.scheduler.Scheduler` (reference `sched::FerriteEngine`, `crates/fe-server/src/ferrite.rs`)."""

    def __init__(self, sched, model_name: str):
        from ..engine.scheduler import Event, Request
        self.sched = sched
        self.model_name = model_name
        self._Request, self._Event = Request, Event
        sched.start()

    def info(self) -> EngineInfo:
        e = self.sched.eng
        return EngineInfo("ferrite", self.model_name, e.ecfg.n_slots, e.ecfg.max_ctx, e.full_cfg.vocab)

    def submit(self, req: GenRequest, sink: TokenSink) -> None:
        def forward(ev):
            sink(GenEvent(ev.kind, list(ev.tokens), ev.reason, dict(ev.timings), ev.message))
        self.sched.submit(self._Request(list(req.ids), req.sampling, forward, list(req.snapshots), req.cancel, req.guard))

    def dead(self) -> Optional[str]:
        return self.sched.dead()

    def incoming(self, delta: int) -> None:
        self.sched.incoming = max(0, self.sched.incoming + delta)

    def load(self) -> Dict[str, int]:
        return {"running": self.sched.running, "queued": self.sched.queued}

    def metrics(self) -> Dict[str, float]:
        return {k: float(v) for k, v in self.sched.stats.items()}

    def shutdown(self) -> None:
        self.sched.stop()


class MockEngine(EngineBase):
    """Scripted replies for protocol tests (reference `MockEngine` / `plan_response`, `crates/fe-server/src/mock.rs`):
    the reply text is planned from the prompt text. Directives inside the last user message:
      `[[reason:TEXT]]` reasoning block, `[[say:TEXT]]` words before the calls, `[[call:NAME:JSON]]` a tool call in the
      JSON body form, `[[xcall:NAME:JSON]]` the same call in the XML parameter form, `[[repeat:N:TEXT]]` TEXT N times
      (long writes, loops), `[[burst:N]]` tokens per event, `[[slow:MS]]` a pause before the first token (slow prefill),
      `[[silent]]` never answers (watchdog test), `[[die]]` reports the engine dead, otherwise echoes the message.
      The prompt tokens shared with the previous request's prompt are reported as served from the cache."""

    def __init__(self, tokenizer, model_name: str = "mock", max_batch: int = 4, max_len: int = 8192, delay_s: float = 0.0):
        self.tok = tokenizer
        self.model_name = model_name
        self.max_batch, self.max_len, self.delay = max_batch, max_len, delay_s
        self._dead: Optional[str] = None
        self._running = 0
        self._lock = threading.Lock()
        self.sem = threading.Semaphore(max_batch)
        self._last_prompt: List[int] = []

    def info(self) -> EngineInfo:
        return EngineInfo("mock", self.model_name, self.max_batch, self.max_len, self.tok.vocab_size)

    def dead(self) -> Optional[str]:
        return self._dead

    def load(self) -> Dict[str, int]:
        return {"running": self._running, "queued": 0}

    @staticmethod
    def plan_response(prompt_text: str) -> Dict[str, Any]:
        import re
        last = prompt_text.rsplit("<|im_start|>user\n", 1)[-1].split("<|im_end|>")[0]
        plan = {"burst": 1, "silent": "[[silent]]" in last, "die": "[[die]]" in last, "text": "", "slow_ms": 0}
        out = ""
        m = re.search(r"\[\[reason:(.*?)\]\]", last, re.S)
        thinking_open = prompt_text.rstrip().endswith("<think>")
        if m:
            out += ("" if thinking_open else "<think>\n") + m.group(1) + "\n</think>\n\n"
        elif thinking_open:
            out += "\n</think>\n\n"
        m = re.search(r"\[\[say:(.*?)\]\]", last, re.S)
        if m:
            out += m.group(1) + "\n"
        for kind, name, js in re.findall(r"\[\[(x?call):([^:\]]+):(.*?)\]\]", last, re.S):
            if kind == "call":
                out += "<tool_call>\n{\"name\": \"" + name + "\", \"arguments\": " + js + "}\n</tool_call>\n"
            else:
                import json as _json
                out += "<tool_call>\n<function=" + name + ">\n"
                for k, v in _json.loads(js).items():
                    out += "<parameter=" + k + ">\n" + (v if isinstance(v, str) else _json.dumps(v, ensure_ascii=False)) + "\n</parameter>\n"
                out += "</function>\n</tool_call>\n"
        m = re.search(r"\[\[repeat:(\d+):(.*?)\]\]", last, re.S)
        if m:
            out += m.group(2) * int(m.group(1))
        m = re.search(r"\[\[burst:(\d+)\]\]", last)
        if m:
            plan["burst"] = int(m.group(1))
        m = re.search(r"\[\[slow:(\d+)\]\]", last)
        if m:
            plan["slow_ms"] = int(m.group(1))
        plain = re.sub(r"\[\[.*?\]\]", "", last, flags=re.S).strip()
        if plain and "call:" not in last and "[[repeat:" not in last:
            out += "echo: " + plain
        plan["text"] = out
        return plan

    def submit(self, req: GenRequest, sink: TokenSink) -> None:
        threading.Thread(target=self._serve, args=(req, sink), daemon=True).start()

    def _serve(self, req: GenRequest, sink: TokenSink) -> None:
        with self.sem:
            with self._lock:
                self._running += 1
            try:
                plan = self.plan_response(self.tok.decode(req.ids))
                if plan["die"]:
                    self._dead = "mock engine told to die"
                    sink(GenEvent("error", message=self._dead))
                    return
                if plan["silent"]:
                    while not req.cancel.is_set():
                        time.sleep(0.01)
                    sink(GenEvent("finish", reason="cancelled"))
                    return
                with self._lock:                       # a one-entry prefix cache: what the prompt shares with the last one
                    cached = 0
                    for a, b in zip(req.ids, self._last_prompt):
                        if a != b:
                            break
                        cached += 1
                    self._last_prompt = list(req.ids)
                if plan["slow_ms"]:
                    req.cancel.wait(plan["slow_ms"] / 1e3)
                ids = self.tok.encode(plan["text"])[:req.sampling.max_tokens]
                t0 = time.time()
                reason = "stop" if len(ids) < req.sampling.max_tokens else "length"
                for i in range(0, len(ids), plan["burst"]):
                    if req.cancel.is_set():
                        reason = "cancelled"
                        break
                    chunk = ids[i:i + plan["burst"]]
                    if req.guard is not None:
                        g = req.guard(chunk)
                        if g:
                            sink(GenEvent("tokens", tokens=chunk))
                            reason = g
                            break
                    sink(GenEvent("tokens", tokens=chunk))
                    if self.delay:
                        time.sleep(self.delay)
                sink(GenEvent("finish", reason=reason, timings={
                    "prompt_n": len(req.ids), "cache_n": min(cached, max(0, len(req.ids) - 1)), "prompt_ms": 0.0, "predicted_n": len(ids),
                    "predicted_ms": 1e3 * (time.time() - t0)}))
            finally:
                with self._lock:
                    self._running -= 1
