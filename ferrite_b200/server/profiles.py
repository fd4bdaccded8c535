"""Sampling defaults per phase: `sampling.<profile>.json` beside the model fills every field a request leaves out, and
the effective values are echoed to the client in the `x-sampling-effective` header. Counterpart of `GenDefaults` /
`PhaseDefaults::from_dir` and `resolve_sampling` (`crates/fe-server/src/server.rs:467`)."""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Optional

from .api import SamplingRequest


@dataclass
class PhaseDefaults:
    temperature: float = 0.7
    top_p: float = 0.8
    top_k: int = 20
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 4096


@dataclass
class GenDefaults:
    thinking: PhaseDefaults = field(default_factory=lambda: PhaseDefaults(temperature=0.6, top_p=0.95))
    non_thinking: PhaseDefaults = field(default_factory=PhaseDefaults)
    max_reasoning_tokens: Optional[int] = None
    no_token_timeout_s: float = 60.0
    reply_wall_limit_s: float = 0.0
    loop_breaker: bool = True
    loop_rules: Optional[Dict[str, Any]] = None        # thresholds of the loop breaker (`loopdet.LoopCfg.from_json`)

    @staticmethod
    def from_dir(model_dir: Optional[str], profile: str = "default") -> "GenDefaults":
        g = GenDefaults()
        if not model_dir:
            return g
        gc = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(gc):
            d = json.load(open(gc))
            for ph in (g.thinking, g.non_thinking):
                for k in ("temperature", "top_p", "top_k", "repetition_penalty"):
                    if k in d and d[k] is not None:
                        setattr(ph, k, type(getattr(ph, k))(d[k]))
        for name in (f"sampling.{profile}.json", "sampling.json"):
            p = os.path.join(model_dir, name)
            if os.path.exists(p):
                d = json.load(open(p))
                for phase, obj in (("thinking", g.thinking), ("non_thinking", g.non_thinking)):
                    for k, v in (d.get(phase) or {}).items():
                        if hasattr(obj, k):
                            setattr(obj, k, v)
                for k in ("max_reasoning_tokens", "no_token_timeout_s", "reply_wall_limit_s", "loop_breaker", "loop_rules"):
                    if k in d:
                        setattr(g, k, d[k])
                break
        return g


def resolve_sampling(req: SamplingRequest, defaults: GenDefaults, thinking: bool, ctx_left: int) -> Dict[str, Any]:
    """Request fields win; omitted ones come from the phase profile. Returns the effective settings."""
    ph = defaults.thinking if thinking else defaults.non_thinking
    eff = asdict(ph)
    for k in ("temperature", "top_p", "top_k", "min_p", "presence_penalty", "frequency_penalty", "repetition_penalty",
              "max_tokens"):
        v = getattr(req, k)
        if v is not None:
            eff[k] = v
    eff["max_tokens"] = max(1, min(int(eff["max_tokens"]), ctx_left))
    eff["seed"] = req.seed
    eff["phase"] = "thinking" if thinking else "non_thinking"
    return eff
