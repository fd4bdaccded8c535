"""Loop breaker and per-request phase bookkeeping (reasoning cap, loop rules) for thinking-aware serving.

A loop is an EXACT token cycle that reaches the current position: the tail of the output is periodic. A rule fires only
when the periodic tail holds a minimum number of full repeats of the cycle AND a minimum number of repeated tokens
(tokens beyond the first occurrence), so short cycles need many repeats and long ones few. Text that says something two
or three times and moves on, spans that are similar but not identical, and lines that differ by a counter never match;
those wandering loops are the repeated-sentence rule's job, which works on the decoded text.

Phases and what a firing does (behaviour of the reference's `PhaseTracker`, `crates/fe-server/src/loopdet.rs:452-700`;
thresholds `LoopCfg` `:20-40,247-262`, sentence rule `SentCfg` / `SentDet` `:42-245`, cycle finder `LoopDet` `:307-392`):

* reasoning (until the `</think>` token): the cap or a loop closes the block (`Trig.CLOSE`: the engine appends
  `</think>` and the model answers);
* answer: the first firing boosts the sampling for `BOOST_TOKENS` tokens, a second one ends the request (`Trig.END_LOOP`);
* tool call (after a call mark): much higher thresholds, since argument values (files with identical rows) repeat
  legitimately; with recovery on, the first firing asks for a rewind to where the cycle began (`Trig.REWIND`).
"""
from __future__ import annotations

import json
import os
import re
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple

BOOST_TOKENS = 96          # tokens of boosted sampling after the first answer-phase firing
SENT_BATCH = 16            # tokens the repeated-sentence rule decodes at a time
NGRAM = 12                 # tokens hashed to propose a period
UNIT_MIN_CHARS = 4         # letters or digits a text unit needs to enter the sentence window


@dataclass
class LoopRule:
    min_repeats: int
    min_repeated_tokens: int


@dataclass
class SentCfg:
    enabled: bool = True
    window: int = 64
    min_chars: int = 16
    min_count: int = 3
    min_fraction: float = 0.7
    min_tokens: int = 600
    answer_min_tokens: int = 1200

    @staticmethod
    def from_json(v: Optional[Dict[str, Any]]) -> "SentCfg":
        c = SentCfg()
        if isinstance(v, dict):
            for k in ("window", "min_chars", "min_count", "min_tokens", "answer_min_tokens"):
                if isinstance(v.get(k), (int, float)):
                    setattr(c, k, max(1, int(v[k])))
            if isinstance(v.get("min_fraction"), (int, float)):
                c.min_fraction = min(1.0, max(0.0, float(v["min_fraction"])))
            if isinstance(v.get("enabled"), bool):
                c.enabled = v["enabled"]
        return c


@dataclass
class LoopCfg:
    min_period: int = 1
    max_period: int = 512
    reasoning: LoopRule = field(default_factory=lambda: LoopRule(4, 400))
    answer: LoopRule = field(default_factory=lambda: LoopRule(8, 400))
    call: LoopRule = field(default_factory=lambda: LoopRule(30, 3000))
    sentence: SentCfg = field(default_factory=SentCfg)
    call_recover: bool = False
    recover_temperature: float = 0.7
    recover_top_p: float = 0.95

    @staticmethod
    def from_json(v: Optional[Dict[str, Any]]) -> "LoopCfg":
        """Defaults overlaid with the keys present (`loop_rules` of a sampling profile; the environment variable
        FE_LOOP_RULES, the same JSON object, overrides it)."""
        env = os.environ.get("FE_LOOP_RULES")
        if env:
            try:
                v = json.loads(env)
            except json.JSONDecodeError:
                pass
        c = LoopCfg()
        if not isinstance(v, dict):
            return c
        num = lambda j, k: int(j[k]) if isinstance(j.get(k), (int, float)) else None
        if num(v, "min_period") is not None:
            c.min_period = max(1, num(v, "min_period"))
        if num(v, "max_period") is not None:
            c.max_period = max(c.min_period, num(v, "max_period"))
        for k in ("reasoning", "answer", "call"):
            j = v.get(k)
            if isinstance(j, dict):
                r = getattr(c, k)
                if num(j, "min_repeats") is not None:
                    r.min_repeats = max(2, num(j, "min_repeats"))
                if num(j, "min_repeated_tokens") is not None:
                    r.min_repeated_tokens = max(0, num(j, "min_repeated_tokens"))
        c.sentence = SentCfg.from_json(v.get("sentence"))
        if isinstance(v.get("call_recover"), bool):
            c.call_recover = v["call_recover"]
        return c

    def fires(self, r: LoopRule, cyc: "Cycle") -> bool:
        return (self.min_period <= cyc.period <= self.max_period and cyc.repeats >= r.min_repeats
                and cyc.repeated_tokens >= r.min_repeated_tokens)


@dataclass
class Cycle:
    period: int
    repeated_tokens: int       # tail tokens that each equal the token `period` positions before them

    @property
    def repeats(self) -> int:
        return self.repeated_tokens // self.period + 1


class LoopDet:
    """Period of the tail of a token stream, one token at a time. While the tail is periodic the period is tracked with
    one comparison per token. When it is not, the position where the last NGRAM tokens were last seen proposes a period
    (their distance), which is verified by comparing tokens backwards; an n-gram that occurs twice inside one cycle
    proposes a distance that is not a period and fails the comparison."""

    def __init__(self, max_period: int = 512):
        self.max_period = max_period
        self.restart()

    def restart(self) -> None:
        self.toks: List[int] = []
        self.period = 0
        self.run = 0
        self.seen: Dict[Tuple[int, ...], int] = {}

    def push(self, t: int) -> None:
        toks = self.toks
        toks.append(int(t))
        n = len(toks)
        if self.period and toks[n - 1] == toks[n - 1 - self.period]:
            self.run += 1
        else:
            self.period = self.run = 0
        if n >= NGRAM:
            key = tuple(toks[n - NGRAM:])
            prev = self.seen.get(key)
            self.seen[key] = n
            if self.period == 0 and prev is not None:
                p = n - prev
                if 0 < p <= self.max_period:
                    run = 0
                    i = n - 1
                    while i - p >= 0 and toks[i] == toks[i - p]:
                        run += 1
                        i -= 1
                    if run >= max(p, NGRAM):
                        self.period, self.run = p, run
        elif n >= 2 and self.period == 0:
            # very short streams: a run of one token (period 1) is found directly
            if toks[n - 1] == toks[n - 2]:
                self.period, self.run = 1, 1
        if len(self.seen) > 1 << 16:
            cut = n - 4 * self.max_period
            self.seen = {k: v for k, v in self.seen.items() if v >= cut}

    def cycle(self) -> Optional[Cycle]:
        return Cycle(self.period, self.run) if self.period else None

    def cycle_ids(self) -> List[int]:
        return self.toks[len(self.toks) - self.period:] if self.period else []


@dataclass
class SentHit:
    distinct: int          # distinct recurring units in the window
    tokens: int            # tokens over which the window stayed saturated
    sample: str            # the most frequent unit


_SPLIT = re.compile(r"(?<=[.!?])\s+|\n+")


class SentDet:
    """The repeated-sentence rule: text in, a hit when the same few sentences keep coming back (see `SentCfg`)."""

    def __init__(self, cfg: SentCfg):
        self.cfg = cfg
        self.restart()

    def restart(self) -> None:
        self.partial = ""
        self.fence = False
        self.win: Deque[Tuple[str, int]] = deque()      # (normalised unit, token count when it ended)
        self.tokens = 0
        self.sat_since: Optional[int] = None

    def in_fence(self) -> bool:
        return self.fence

    @staticmethod
    def normalise(unit: str) -> str:
        return "".join(ch.lower() for ch in unit if ch.isalnum())

    def _units(self, text: str, final: bool = False) -> List[str]:
        buf = self.partial + text
        out: List[str] = []
        lines = buf.split("\n")
        self.partial = "" if final else lines.pop()
        for line in lines:
            if line.strip().startswith("```"):
                self.fence = not self.fence
                continue
            if self.fence:
                continue
            out.extend(u for u in _SPLIT.split(line) if u)
        return out

    def push_text(self, text: str, ntok: int, min_tokens: int) -> Optional[SentHit]:
        self.tokens += ntok
        for u in self._units(text):
            key = self.normalise(u)
            if len(key) < UNIT_MIN_CHARS:
                continue
            self.win.append((key, self.tokens))
            while len(self.win) > self.cfg.window:
                self.win.popleft()
        if len(self.win) < self.cfg.window:
            self.sat_since = None
            return None
        counts: Dict[str, int] = {}
        for k, _ in self.win:
            counts[k] = counts.get(k, 0) + 1
        recurring = {k: c for k, c in counts.items() if len(k) >= self.cfg.min_chars and c >= self.cfg.min_count}
        n = sum(recurring.values())
        if n < self.cfg.min_fraction * self.cfg.window:
            self.sat_since = None
            return None
        if self.sat_since is None:
            self.sat_since = self.win[0][1]
        span = self.tokens - self.sat_since
        if span < min_tokens:
            return None
        best = max(recurring, key=recurring.get)
        return SentHit(len(recurring), span, best)


class Trig(Enum):
    NONE = 0
    CLOSE = 1          # close the reasoning block (cap or loop) and let the model answer
    REWIND = 2         # tool-call cycle with recovery on: take back `PhaseTracker.rewind` = (tokens, of them held back)
    END_LOOP = 3       # an answer-phase loop that came back after the sampling boost: end the request cleanly


@dataclass
class PhaseEvents:
    reasoning_tokens: int = 0
    reasoning_capped: bool = False
    loop_breaks: int = 0
    sentence_breaks: int = 0
    rewinds: int = 0


def has_call_mark(toks: Sequence[int], marks: Sequence[Sequence[int]]) -> bool:
    """Does `toks` hold one of the marks in its last 64 tokens?"""
    w = list(toks[-64:])
    for m in marks:
        k = len(m)
        if k and any(w[i:i + k] == list(m) for i in range(len(w) - k + 1)):
            return True
    return False


class PhaseTracker:
    """Per-request phase state: where the generation is (reasoning / answer / tool call), the reasoning cap and the loop
    breaker. Engine-independent: feed it every generated token (a forced `</think>` included) and act on the `Trig`."""

    def __init__(self, think_end: Optional[int], in_reasoning: bool, max_reasoning: Optional[int] = None,
                 loop_breaker: bool = True, rules: Optional[LoopCfg] = None, call_marks: Sequence[Sequence[int]] = (),
                 detok: Optional[Callable[[Sequence[int]], str]] = None):
        self.think_end = think_end
        self.cap = max_reasoning if (max_reasoning and max_reasoning > 0) else 0
        self.breaker = loop_breaker
        self.rules = rules or LoopCfg()
        self.call_marks = [list(m) for m in call_marks if m]
        self.in_reasoning = bool(in_reasoning and think_end is not None)
        self.in_call = False
        self.generated: List[int] = []
        self.boost_until = 0
        self.boosts = 0
        self.recover_on = False
        self.hold_from: Optional[int] = None
        self.recovering = False
        self.rewind: Tuple[int, int] = (0, 0)
        self.det = LoopDet(self.rules.max_period)
        self.detok = detok
        self.sent = SentDet(self.rules.sentence) if (detok is not None and self.rules.sentence.enabled) else None
        self.pend: List[int] = []
        self.sent_hit: Optional[SentHit] = None
        self.events = PhaseEvents()

    # ---- state ----------------------------------------------------------------------------------------------------
    def boosting(self) -> bool:
        return len(self.generated) < self.boost_until

    def holding(self) -> bool:
        """Tokens generated since a tool-call cycle was first seen are held back from the client."""
        return self.hold_from is not None

    def enable_recover(self, force: bool = False) -> None:
        self.recover_on = force or self.rules.call_recover

    def _rule(self) -> LoopRule:
        return self.rules.call if self.in_call else (self.rules.reasoning if self.in_reasoning else self.rules.answer)

    def _restart_detectors(self) -> None:
        self.det.restart()
        if self.sent is not None:
            self.sent.restart()
        self.pend = []
        self.sent_hit = None

    def _feed_sentences(self, flush: bool = False) -> None:
        if self.sent is None or self.in_call:
            self.pend = []
            return
        if len(self.pend) < SENT_BATCH and not flush:
            return
        text = self.detok(self.pend)
        if text.endswith("�") and not flush:        # a split UTF-8 sequence: wait for its rest
            return
        n, self.pend = len(self.pend), []
        min_tokens = self.rules.sentence.min_tokens if self.in_reasoning else self.rules.sentence.answer_min_tokens
        hit = self.sent.push_text(text, n, min_tokens)
        if hit is not None:
            self.sent_hit = hit

    # ---- feeding --------------------------------------------------------------------------------------------------
    def feed(self, toks: Sequence[int]) -> Trig:
        trig = Trig.NONE
        for t in toks:
            t = int(t)
            self.generated.append(t)
            if self.in_reasoning:
                self.events.reasoning_tokens += 1
                if t == self.think_end:
                    self.in_reasoning = False
                    self._restart_detectors()
                    continue
            if not self.in_call and self.call_marks and has_call_mark(self.generated, self.call_marks):
                self.in_call = True
                self._restart_detectors()
            self.det.push(t)
            self.pend.append(t)
            self._feed_sentences()
            if self.in_reasoning and self.cap and self.events.reasoning_tokens >= self.cap:
                self.events.reasoning_capped = True
                self.in_reasoning = False
                self._restart_detectors()
                trig = Trig.CLOSE
                continue
            if not self.breaker or self.boosting():
                continue
            cyc = self.det.cycle()
            fired = cyc is not None and self.rules.fires(self._rule(), cyc)
            sent_fired = self.sent_hit is not None and not self.in_call
            if self.in_call and self.recover_on and cyc is not None and self.hold_from is None and cyc.repeated_tokens >= cyc.period:
                self.hold_from = len(self.generated) - cyc.repeated_tokens + cyc.period     # the cycle has been seen twice
            if not (fired or sent_fired):
                if cyc is None:
                    self.hold_from = None
                continue
            self.events.loop_breaks += 1
            if sent_fired and not fired:
                self.events.sentence_breaks += 1
            if self.in_reasoning:
                self.in_reasoning = False
                self._restart_detectors()
                trig = Trig.CLOSE
            elif self.in_call and self.recover_on and not self.recovering and cyc is not None:
                back = cyc.repeated_tokens + cyc.period
                held = len(self.generated) - (self.hold_from if self.hold_from is not None else len(self.generated))
                back = min(back, len(self.generated))
                self.rewind = (back, min(held, back))
                del self.generated[len(self.generated) - back:]
                self.recovering = True
                self.hold_from = None
                self.events.rewinds += 1
                self._restart_detectors()
                return Trig.REWIND
            elif self.boosts == 0 and not self.in_call:
                self.boosts = 1
                self.boost_until = len(self.generated) + BOOST_TOKENS
                self._restart_detectors()
            else:
                return Trig.END_LOOP
        return trig

    def cycle_preview(self) -> str:
        """First 80 characters of the cycle, for a log line."""
        ids = self.det.cycle_ids()
        return (self.detok(ids) if self.detok else " ".join(map(str, ids)))[:80]
