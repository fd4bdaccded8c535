"""Reply guard of one request: adapts the phase tracker (`loopdet.PhaseTracker`: reasoning cap, loop rules,
repeated-sentence rule) to the scheduler's guard hook. Counterpart of the reference's `PhaseGuard::feed`
(`crates/fe-server/src/guard.rs:106`) and of the guard built in `crates/fe-server/src/ferrite.rs` (`guard(&params)`):

* the cap, or a loop inside the reasoning block, forces the block's closing tokens so the model answers;
* the first loop in the answer boosts the sampling (temperature 0.7, top-p 0.95: a greedy request leaves its cycle) for
  `BOOST_TOKENS` tokens, then the request's own sampling comes back; a loop that returns ends the reply;
* what fired is kept in `events` (reported with the finish and in the request-capture file).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from .loopdet import BOOST_TOKENS, LoopCfg, PhaseEvents, PhaseTracker, Trig

__all__ = ["BOOST_TOKENS", "GuardAction", "PhaseGuard"]


@dataclass
class GuardAction:
    force_tokens: List[int] = field(default_factory=list)   # tokens to append to the sequence (the block's closing tag)
    finish: Optional[str] = None                            # end the reply with this reason
    boost: bool = False                                     # the boosted stretch is on
    boost_started: bool = False                             # ... and began with these tokens
    boost_ended: bool = False                               # the request's own sampling is back


class PhaseGuard:
    """think_end_ids: the tokens of `</think>` as the model writes it (detection); close_ids: what is forced to close a
    capped or looping block (defaults to think_end_ids). A multi-token `</think>` (byte-level tokenizers) is detected
    on its last token, with the tokens before it compared."""

    def __init__(self, think_end_ids: Sequence[int], in_thinking: bool, max_reasoning: Optional[int] = None,
                 loop_breaker: bool = True, rules: Optional[LoopCfg] = None, close_ids: Optional[Sequence[int]] = None,
                 call_marks: Sequence[Sequence[int]] = (), detok: Optional[Callable[[Sequence[int]], str]] = None):
        self.think_end = [int(t) for t in think_end_ids]
        self.close_ids = [int(t) for t in (close_ids if close_ids is not None else think_end_ids)]
        last = self.think_end[-1] if self.think_end else None
        self.tracker = PhaseTracker(last, in_thinking, max_reasoning, loop_breaker, rules, call_marks, detok)
        self.tail: List[int] = []
        self.was_boosting = False

    @property
    def in_thinking(self) -> bool:
        return self.tracker.in_reasoning

    @property
    def events(self) -> PhaseEvents:
        return self.tracker.events

    def feed(self, toks: Sequence[int], text: str = "") -> GuardAction:
        act = GuardAction()
        tr = self.tracker
        for t in toks:
            t = int(t)
            k = len(self.think_end)
            if tr.in_reasoning and k > 1 and t == self.think_end[-1]:
                # the last token of the tag only counts when the tokens before it are the tag's
                if self.tail[-(k - 1):] != self.think_end[:-1]:
                    tr.think_end, keep = None, tr.think_end
                    trig = tr.feed([t])
                    tr.think_end = keep
                else:
                    trig = tr.feed([t])
            else:
                trig = tr.feed([t])
            self.tail = (self.tail + [t])[-max(8, k):]
            if trig == Trig.CLOSE:
                act.force_tokens = list(self.close_ids)
            elif trig == Trig.END_LOOP:
                act.finish = "loop"
                break
        now = tr.boosting()
        act.boost = now
        act.boost_started = now and not self.was_boosting
        act.boost_ended = self.was_boosting and not now
        self.was_boosting = now
        return act
