"""OpenAI request types (lenient: unknown fields ignored, nulls allowed) and OpenAI-shaped errors.
Counterpart of `crates/fe-server/src/api.rs` (`ChatRequest`, `CompletionRequest`, `SamplingRequest`, `ApiError`)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ApiError(Exception):
    def __init__(self, status: int, message: str, typ: str = "invalid_request_error", param: Optional[str] = None,
                 code: Optional[str] = None):
        super().__init__(message)
        self.status, self.message, self.typ, self.param, self.code = status, message, typ, param, code

    def body(self) -> Dict[str, Any]:
        return {"error": {"message": self.message, "type": self.typ, "param": self.param, "code": self.code}}


def _num(d, k, typ, lo=None, hi=None):
    v = d.get(k)
    if v is None:
        return None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ApiError(400, f"'{k}' must be a number", param=k)
    if (lo is not None and v < lo) or (hi is not None and v > hi):
        raise ApiError(400, f"'{k}' is out of range", param=k)
    return typ(v)


@dataclass
class SamplingRequest:
    """Sampling fields shared by chat and completions (OpenAI + the common vLLM extensions)."""

    max_tokens: Optional[int] = None
    min_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    presence_penalty: Optional[float] = None
    frequency_penalty: Optional[float] = None
    repetition_penalty: Optional[float] = None
    seed: Optional[int] = None
    stop: List[str] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False
    include_stop_str_in_output: bool = False

    @staticmethod
    def parse(d: Dict[str, Any]) -> "SamplingRequest":
        stop = d.get("stop")
        if stop is None:
            stop = []
        elif isinstance(stop, str):
            stop = [stop]
        elif not (isinstance(stop, list) and all(isinstance(s, str) for s in stop)):
            raise ApiError(400, "'stop' must be a string or a list of strings", param="stop")
        mt = _num(d, "max_completion_tokens", int, 1) or _num(d, "max_tokens", int, 1)
        return SamplingRequest(
            max_tokens=mt, min_tokens=_num(d, "min_tokens", int, 0), temperature=_num(d, "temperature", float, 0.0),
            top_p=_num(d, "top_p", float, 0.0, 1.0), top_k=_num(d, "top_k", int), min_p=_num(d, "min_p", float, 0.0, 1.0),
            presence_penalty=_num(d, "presence_penalty", float), frequency_penalty=_num(d, "frequency_penalty", float),
            repetition_penalty=_num(d, "repetition_penalty", float, 0.0), seed=_num(d, "seed", int), stop=stop,
            stop_token_ids=[int(x) for x in (d.get("stop_token_ids") or [])], ignore_eos=bool(d.get("ignore_eos") or False),
            include_stop_str_in_output=bool(d.get("include_stop_str_in_output") or False))


@dataclass
class ChatRequest:
    messages: List[Dict[str, Any]]
    sampling: SamplingRequest
    model: Optional[str] = None
    tools: List[Dict[str, Any]] = field(default_factory=list)
    tool_choice: Any = None
    parallel_tool_calls: bool = True
    stream: bool = False
    include_usage: bool = False
    enable_thinking: Optional[bool] = None
    max_reasoning_tokens: Optional[int] = None
    loop_breaker: Optional[bool] = None
    n: int = 1
    raw: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def parse(d: Any) -> "ChatRequest":
        if not isinstance(d, dict):
            raise ApiError(400, "request body must be a JSON object")
        msgs = d.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise ApiError(400, "'messages' must be a non-empty list", param="messages")
        for m in msgs:
            if not isinstance(m, dict) or "role" not in m:
                raise ApiError(400, "each message needs a 'role'", param="messages")
        tools = d.get("tools") or []
        if not isinstance(tools, list):
            raise ApiError(400, "'tools' must be a list", param="tools")
        if (d.get("n") or 1) != 1:
            raise ApiError(400, "only n = 1 is supported", param="n")
        kw = d.get("chat_template_kwargs") or {}
        so = d.get("stream_options") or {}
        return ChatRequest(
            messages=msgs, sampling=SamplingRequest.parse(d), model=d.get("model"), tools=tools,
            tool_choice=d.get("tool_choice"), parallel_tool_calls=d.get("parallel_tool_calls") is not False,
            stream=bool(d.get("stream") or False), include_usage=bool(so.get("include_usage") or False),
            enable_thinking=kw.get("enable_thinking", d.get("enable_thinking")),
            max_reasoning_tokens=_num(d, "max_reasoning_tokens", int, 0), loop_breaker=d.get("loop_breaker"), raw=d)


@dataclass
class CompletionRequest:
    prompt: Any
    sampling: SamplingRequest
    model: Optional[str] = None
    stream: bool = False
    include_usage: bool = False
    echo: bool = False

    @staticmethod
    def parse(d: Any) -> "CompletionRequest":
        if not isinstance(d, dict):
            raise ApiError(400, "request body must be a JSON object")
        p = d.get("prompt")
        if isinstance(p, list) and len(p) == 1 and isinstance(p[0], str):
            p = p[0]
        if not (isinstance(p, str) or (isinstance(p, list) and all(isinstance(x, int) for x in p))):
            raise ApiError(400, "'prompt' must be a string or a list of token ids", param="prompt")
        so = d.get("stream_options") or {}
        return CompletionRequest(p, SamplingRequest.parse(d), d.get("model"), bool(d.get("stream") or False),
                                 bool(so.get("include_usage") or False), bool(d.get("echo") or False))
