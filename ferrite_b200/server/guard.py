"""Reply guards working on the token / text stream of one request: reasoning cap, exact-cycle loop breaker,
repeated-sentence rule, and the boost-then-end escalation. Counterparts: `PhaseGuard::feed` (`crates/fe-server/src/
guard.rs:106`) over `PhaseTracker`, `SentDet` and the cycle detector of `loopdet.rs`."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

BOOST_TOKENS = 96      # tokens of boosted sampling after a loop is seen before the reply is ended


@dataclass
class LoopRules:
    min_period: int = 4            # shortest token cycle considered
    max_period: int = 256
    repeats: int = 4               # a cycle repeated this many times is a loop
    sentence_repeats: int = 5      # the same sentence this many times is a loop
    min_sentence_chars: int = 24


class CycleDetector:
    """Exact repetition at the tail of the token stream: ... P P P P for some period |P| in [min, max]."""

    def __init__(self, rules: LoopRules):
        self.r = rules
        self.toks: List[int] = []

    def feed(self, toks: Sequence[int]) -> Optional[int]:
        self.toks.extend(int(t) for t in toks)
        t = self.toks
        n = len(t)
        for p in range(self.r.min_period, min(self.r.max_period, n // self.r.repeats) + 1):
            need = p * self.r.repeats
            if n < need:
                break
            tail = t[n - need:]
            if all(tail[i] == tail[i % p] for i in range(need)):
                return p
        if n > 4 * self.r.max_period * self.r.repeats:
            self.toks = t[-2 * self.r.max_period * self.r.repeats:]
        return None


class SentenceDetector:
    """Counts repeated sentences (normalised, long enough) in the decoded text."""

    def __init__(self, rules: LoopRules):
        self.r = rules
        self.buf = ""
        self.counts: Dict[str, int] = {}

    def feed(self, text: str) -> Optional[str]:
        self.buf += text
        hit = None
        while True:
            idx = min((i for i in (self.buf.find(c) for c in ".!?\n") if i >= 0), default=-1)
            if idx < 0:
                break
            sent, self.buf = self.buf[:idx + 1], self.buf[idx + 1:]
            key = " ".join(sent.lower().split())
            if len(key) < self.r.min_sentence_chars:
                continue
            self.counts[key] = self.counts.get(key, 0) + 1
            if self.counts[key] >= self.r.sentence_repeats:
                hit = key
        return hit


@dataclass
class GuardAction:
    force_tokens: List[int] = field(default_factory=list)   # tokens to append to the sequence (e.g. </think>)
    finish: Optional[str] = None                            # end the reply with this reason
    boost: bool = False                                     # raise temperature / penalties for a while


class PhaseGuard:
    """Tracks thinking vs answer phase; caps reasoning length; escalates on loops: first a sampling boost for
    BOOST_TOKENS tokens, and if the loop is still there, the end of the reply."""

    def __init__(self, think_end_ids: Sequence[int], in_thinking: bool, max_reasoning: Optional[int],
                 loop_breaker: bool = True, rules: Optional[LoopRules] = None):
        self.think_end = list(think_end_ids)
        self.in_thinking = in_thinking
        self.max_reasoning = max_reasoning
        self.loop_breaker = loop_breaker
        self.rules = rules or LoopRules()
        self.cycles = CycleDetector(self.rules)
        self.sents = SentenceDetector(self.rules)
        self.n_reasoning = 0
        self.boost_left = 0
        self.loops_seen = 0

    def feed(self, toks: Sequence[int], text: str = "") -> GuardAction:
        act = GuardAction()
        if self.in_thinking:
            self.n_reasoning += len(toks)
        if self.in_thinking and self.think_end:
            joined = self.cycles.toks + [int(t) for t in toks]
            k = len(self.think_end)
            for i in range(max(0, len(joined) - len(toks) - k + 1), len(joined) - k + 1):
                if joined[i:i + k] == self.think_end:
                    self.in_thinking = False
                    break
        if self.in_thinking and self.max_reasoning is not None and self.n_reasoning >= self.max_reasoning:
            act.force_tokens = list(self.think_end)           # close the reasoning block for the model
            self.in_thinking = False
        period = self.cycles.feed(toks)
        sent = self.sents.feed(text) if text else None
        if self.loop_breaker and (period is not None or sent is not None):
            self.loops_seen += 1
            if self.boost_left == 0 and self.loops_seen == 1:
                self.boost_left = BOOST_TOKENS
                act.boost = True
                self.cycles.toks = []
            elif self.boost_left == 0:
                act.finish = "loop"
        if self.boost_left > 0:
            self.boost_left = max(0, self.boost_left - len(toks))
            act.boost = act.boost or self.boost_left > 0
        return act
