"""Tool definitions, JSON-schema coercion of model-written arguments, and `tool_choice` enforcement.
Counterpart of `crates/fe-server/src/toolcall.rs` and the forced-opener logic of `server.rs:580-741`."""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .api import ApiError


def coerce(value: Any, schema: Optional[Dict[str, Any]]) -> Any:
    """Bend a model-written value towards its schema type: "3" -> 3 for integer, "true" -> True, JSON text ->
    object / array; anything that does not convert is left as it is."""
    if not isinstance(schema, dict):
        return value
    t = schema.get("type")
    if isinstance(t, list):
        t = next((x for x in t if x != "null"), None)
    try:
        if t == "integer" and isinstance(value, str):
            return int(value.strip())
        if t == "number" and isinstance(value, str):
            return float(value.strip())
        if t == "boolean" and isinstance(value, str) and value.strip().lower() in ("true", "false"):
            return value.strip().lower() == "true"
        if t in ("object", "array") and isinstance(value, str):
            v = json.loads(value)
            return coerce(v, schema)
        if t == "string" and not isinstance(value, str):
            return json.dumps(value, ensure_ascii=False)
        if t == "object" and isinstance(value, dict):
            props = schema.get("properties") or {}
            return {k: coerce(v, props.get(k)) for k, v in value.items()}
        if t == "array" and isinstance(value, list):
            return [coerce(v, schema.get("items")) for v in value]
    except (ValueError, json.JSONDecodeError):
        return value
    return value


@dataclass
class ForcedCall:
    """Text the generation prompt is made to end with so that the reply is a tool call (reference `ForcedCall`,
    `crates/fe-server/src/parser.rs:37-70`): any tool -> the reply starts with the function's name; a named tool -> the
    reply starts with its parameters."""
    opener: str
    name: Optional[str]

    @staticmethod
    def make(name: Optional[str], dsml: bool = False) -> "ForcedCall":
        if dsml:
            head = "\n\n<｜DSML｜ calls>\n<｜DSML｜ invoke name=\""
            return ForcedCall(head + (f"{name}\">\n" if name else ""), name)
        return ForcedCall("<tool_call>\n<function=" + (f"{name}>\n" if name else ""), name)


class ToolSet:
    def __init__(self, tools: List[Dict[str, Any]]):
        self.tools: Dict[str, Dict[str, Any]] = {}
        for t in tools or []:
            fn = t.get("function") if isinstance(t, dict) else None
            if not isinstance(fn, dict) or not isinstance(fn.get("name"), str):
                raise ApiError(400, "each tool needs function.name", param="tools")
            self.tools[fn["name"]] = fn

    def __bool__(self) -> bool:
        return bool(self.tools)

    def names(self) -> List[str]:
        return list(self.tools)

    def coerce_arguments(self, name: str, args: Any) -> Any:
        fn = self.tools.get(name)
        if fn is None or not isinstance(args, dict):
            return args
        return coerce(args, fn.get("parameters") or {"type": "object"})

    def resolve_choice(self, tool_choice: Any, dsml: bool = False) -> Optional[ForcedCall]:
        """none -> tools are hidden by the caller; auto/None -> free; required -> must open a call;
        {"type":"function","function":{"name":X}} -> must call X."""
        if tool_choice in (None, "auto", "none"):
            return None
        if tool_choice == "required":
            if not self.tools:
                raise ApiError(400, "tool_choice 'required' needs tools", param="tool_choice")
            return ForcedCall.make(None, dsml)
        if isinstance(tool_choice, dict):
            name = (tool_choice.get("function") or {}).get("name")
            if name not in self.tools:
                raise ApiError(400, f"tool_choice names an unknown tool {name!r}", param="tool_choice")
            return ForcedCall.make(name, dsml)
        raise ApiError(400, "unsupported tool_choice", param="tool_choice")
