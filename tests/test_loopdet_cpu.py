"""Loop breaker: exact-cycle finder, threshold rules per phase, the repeated-sentence rule and the phase tracker
(behaviours of the reference's `crates/fe-server/src/loopdet.rs` tests and of its guard tests in `ferrite.rs`)."""
import random

from ferrite_b200.server.loopdet import (BOOST_TOKENS, Cycle, LoopCfg, LoopDet, LoopRule, PhaseTracker, SentCfg, SentDet, Trig,
                                        has_call_mark)

TE = 900


def test_cycle_finder_tracks_the_period_of_the_tail():
    d = LoopDet()
    rng = random.Random(1)
    for _ in range(300):
        d.push(rng.randrange(1000, 2000))
    assert d.cycle() is None
    cyc = [10, 11, 12, 13, 14, 15, 16]
    for i in range(70):
        d.push(cyc[i % 7])
    c = d.cycle()
    assert c is not None and c.period == 7 and c.repeated_tokens >= 70 - 7 - 12 and c.repeats >= 8
    assert sorted(d.cycle_ids()) == cyc
    d.push(5)                                  # the tail is no longer periodic
    assert d.cycle() is None
    # a run of one token
    d = LoopDet()
    for _ in range(40):
        d.push(3)
    assert d.cycle().period == 1 and d.cycle().repeated_tokens == 39
    # a long cycle with a repeated n-gram inside it still resolves to the true period
    inner = list(range(100, 130))
    long_cycle = inner + [7] + inner + [8]
    d = LoopDet()
    for i in range(5 * len(long_cycle)):
        d.push(long_cycle[i % len(long_cycle)])
    assert d.cycle().period == len(long_cycle)


def test_rules_scale_repeats_with_the_period():
    cfg = LoopCfg()
    r = cfg.reasoning
    assert not cfg.fires(r, Cycle(5, 300)) and cfg.fires(r, Cycle(5, 400))          # 81 repeats of a 5-token cycle
    assert cfg.fires(r, Cycle(300, 900)) and not cfg.fires(r, Cycle(300, 800))      # 4 repeats of a 300-token cycle
    assert not cfg.fires(r, Cycle(600, 5000))                                       # longer than max_period
    c = LoopCfg.from_json({"max_period": 64, "answer": {"min_repeats": 1, "min_repeated_tokens": 10}, "sentence": {"window": 8}})
    assert c.max_period == 64 and c.answer.min_repeats == 2 and c.answer.min_repeated_tokens == 10 and c.sentence.window == 8
    assert has_call_mark([1, 2, 3, 4, 5], [[3, 4]]) and not has_call_mark([1, 2, 3], [[3, 4]])


def test_reasoning_cap_and_cycle_close_the_block():
    t = PhaseTracker(TE, True, max_reasoning=5)
    assert t.feed([1, 2, 3, 4]) == Trig.NONE and t.feed([5]) == Trig.CLOSE
    assert t.events.reasoning_capped and not t.in_reasoning
    assert t.feed([TE, 6, 7]) == Trig.NONE
    # a cycle inside the block closes it; the model's own </think> ends it silently
    t = PhaseTracker(TE, True, rules=LoopCfg(reasoning=LoopRule(4, 60)))
    out = [t.feed([10 + i % 5]) for i in range(200)]
    assert Trig.CLOSE in out and t.events.loop_breaks == 1 and not t.in_reasoning
    t = PhaseTracker(TE, True, max_reasoning=100)
    assert t.feed([1, 2, TE, 3, 4]) == Trig.NONE and not t.in_reasoning and t.events.reasoning_tokens == 3


def test_answer_cycle_boosts_then_ends():
    t = PhaseTracker(None, False, rules=LoopCfg(answer=LoopRule(4, 150)))
    acts = []
    for i in range(2000):
        was = t.boosting()
        tr = t.feed([10 + i % 5])
        if t.boosting() != was:
            acts.append((i + 1, "boost" if t.boosting() else "back"))
        if tr == Trig.END_LOOP:
            acts.append((i + 1, "end"))
            break
    assert [a for _, a in acts] == ["boost", "back", "end"], acts
    assert acts[0][0] < 200 and acts[1][0] == acts[0][0] + BOOST_TOKENS
    assert t.events.loop_breaks == 2


def test_tool_call_phase_uses_its_own_thresholds_and_can_rewind():
    marks = [[50, 51]]
    rules = LoopCfg(answer=LoopRule(4, 40), call=LoopRule(6, 120))
    t = PhaseTracker(None, False, rules=rules, call_marks=marks)
    t.feed([1, 2, 50, 51])
    assert t.in_call
    n = 0
    for i in range(100):                       # 100 repeated tokens: over the answer rule, under the call rule
        assert t.feed([20 + i % 4]) == Trig.NONE
    t = PhaseTracker(None, False, rules=rules, call_marks=marks)
    t.enable_recover(True)
    t.feed([1, 2, 50, 51])
    trig = Trig.NONE
    for i in range(400):
        trig = t.feed([20 + i % 4])
        if trig != Trig.NONE:
            break
    assert trig == Trig.REWIND and t.events.rewinds == 1
    back, held = t.rewind
    assert back >= 120 and 0 < held <= back and len(t.generated) == 4 + i + 1 - back


def test_repeated_sentence_rule():
    cfg = SentCfg(window=16, min_chars=12, min_count=3, min_fraction=0.7, min_tokens=40)
    d = SentDet(cfg)
    sents = ["Let me reconsider the second option again.", "Perhaps the first approach was right after all.",
             "But wait, the constraint rules that out.", "So we are back to the second option."]
    hit = None
    for i in range(60):
        hit = d.push_text(f"{i}. " + sents[i % 4] + "\n", 12, cfg.min_tokens) or hit
    assert hit is not None and hit.distinct == 4 and hit.tokens >= 40
    # an enumeration whose items differ, code inside a fence and short units never saturate
    d = SentDet(cfg)
    for i in range(60):
        assert d.push_text(f"Item {i}: the value of entry number {i * 7919} is {i * i}.\n", 12, cfg.min_tokens) is None
    d = SentDet(cfg)
    d.push_text("```python\n", 3, cfg.min_tokens)
    for i in range(60):
        assert d.push_text("    result.append(compute_value(x))\n", 8, cfg.min_tokens) is None
    assert d.in_fence()


def test_tracker_with_the_sentence_rule_closes_wandering_reasoning():
    vocab = {}
    def tok(s):
        return [vocab.setdefault(w, 1000 + len(vocab)) for w in s.split(" ")]
    inv = lambda ids: " ".join(next(k for k, v in vocab.items() if v == i) for i in ids)
    rules = LoopCfg(sentence=SentCfg(window=12, min_chars=12, min_count=3, min_fraction=0.7, min_tokens=60))
    t = PhaseTracker(TE, True, rules=rules, detok=inv)
    sents = ["Maybe the answer is forty two.\n", "No that cannot be right because of the sign.\n",
             "Let me check the sign once more.\n"]
    trig = Trig.NONE
    for i in range(120):
        # changing labels keep the token stream from being an exact cycle
        trig = t.feed(tok(f"{i}. " + sents[i % 3]))
        if trig != Trig.NONE:
            break
    assert trig == Trig.CLOSE and t.events.sentence_breaks == 1
