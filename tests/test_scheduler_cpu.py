"""Scheduler policy on the CPU engine: continuous batching, prompt-cache resume, parking, speculation, sampling,
fault bookkeeping. Every comparison is against plain single-request greedy decoding of the same tiny model."""
import pytest
import torch

from ferrite_b200.config import EngineConfig, ModelConfig, tiny_hybrid
from ferrite_b200.engine.copy import Copier
from ferrite_b200.engine.engine import Engine
from ferrite_b200.engine.pcache import Park, SlotCache, Snap, common_prefix
from ferrite_b200.engine.sampler import Sampler, Sampling, SplitMix64, dist
from ferrite_b200.engine.scheduler import Event, Request, SchedOptions, Scheduler, generate
from ferrite_b200.models.weights import init_weights


def _engine(n_slots=2, max_ctx=256, chunk=32):
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    return cfg, w, Engine(cfg, w, EngineConfig(n_slots=n_slots, max_ctx=max_ctx, prefill_chunk=chunk), device="cpu")


def _prompt(cfg, n, seed):
    return torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _plain(cfg, w, prompt, n):
    return Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256), device="cpu").generate(prompt, n)


def test_batched_requests_equal_single_greedy():
    cfg, w, eng = _engine(n_slots=2)
    prompts = [_prompt(cfg, 20, 1), _prompt(cfg, 45, 2), _prompt(cfg, 7, 3)]       # 3 requests on 2 slots
    outs = generate(Scheduler(eng), prompts, Sampling(max_tokens=12))
    for p, o in zip(prompts, outs):
        assert o == _plain(cfg, w, p, 12)


def test_prompt_cache_resume_is_exact_and_counts_cached_tokens():
    cfg, w, eng = _engine(n_slots=1)
    sched = Scheduler(eng)
    system = _prompt(cfg, 40, 5)
    turn1 = system + _prompt(cfg, 10, 6)
    o1 = generate(sched, [turn1], Sampling(max_tokens=8), snapshots=[[40, len(turn1)]])[0]
    turn2 = turn1 + o1 + _prompt(cfg, 9, 7)
    o2 = generate(sched, [turn2], Sampling(max_tokens=8), snapshots=[[40, len(turn2)]])[0]
    assert sched.stats["cached_tokens"] >= len(turn1)            # second turn resumed past the first prompt
    assert o2 == _plain(cfg, w, turn2, 8)
    # a different conversation sharing only the system prompt resumes at the pinned system snapshot
    other = system + _prompt(cfg, 12, 8)
    before = sched.stats["cached_tokens"]
    o3 = generate(sched, [other], Sampling(max_tokens=6), snapshots=[[40]])[0]
    assert sched.stats["cached_tokens"] - before == 40
    assert o3 == _plain(cfg, w, other, 6)


def test_parked_sequence_is_restored_into_another_slot():
    cfg, w, eng = _engine(n_slots=1)
    sched = Scheduler(eng)
    a = _prompt(cfg, 70, 11)
    generate(sched, [a], Sampling(max_tokens=4), snapshots=[[64]])
    b = _prompt(cfg, 30, 12)
    generate(sched, [b], Sampling(max_tokens=4))                  # evicts a's sequence to the park pool
    assert len(sched.park) >= 1
    before = sched.stats["cached_tokens"]
    a2 = a + _prompt(cfg, 5, 13)
    out = generate(sched, [a2], Sampling(max_tokens=6))[0]
    assert sched.stats["cached_tokens"] - before == 64            # resumed from the parked snapshot (page move)
    assert out == _plain(cfg, w, a2, 6)


def test_copy_speculation_keeps_greedy_output():
    cfg, w, eng = _engine(n_slots=2)
    span = _prompt(cfg, 12, 21)
    prompt = span * 5                                             # repeated spans: the copier has proposals
    sched = Scheduler(eng, SchedOptions(spec=8))
    out = generate(sched, [prompt, _prompt(cfg, 18, 22)], Sampling(max_tokens=16))
    assert out[0] == _plain(cfg, w, prompt, 16)
    assert out[1] == _plain(cfg, w, _prompt(cfg, 18, 22), 16)
    assert sched.stats["drafted"] > 0


def test_block_drafter_keeps_greedy_output():
    from ferrite_b200.models.drafter import BlockDrafter
    cfg, w, eng = _engine(n_slots=1)
    cfg.tap_layers = [1, 3]
    eng.cfg.tap_layers = [1, 3]
    eng.ex.cfg.tap_layers = [1, 3]
    dcfg = ModelConfig(name="tiny-drafter", hidden=128, inter=256, n_layers=2, full_attn_every=1, head_dim=32, n_q=4,
                       n_kv=2, rotary_dim=32, attn_gate=False, vocab=cfg.vocab, tie_embeddings=True)
    dr = BlockDrafter(dcfg, target_hidden=cfg.hidden, n_taps=2, n_slots=1, max_ctx=256, device="cpu", block=6)
    sched = Scheduler(eng, SchedOptions(spec=6, copy_rows=False), drafter=dr)
    prompt = _prompt(cfg, 25, 31)
    out = generate(sched, [prompt], Sampling(max_tokens=14))[0]
    assert out == _plain(cfg, w, prompt, 14)
    assert sched.stats["drafted"] > 0


def test_sampling_is_seeded_and_respects_filters():
    cfg, w, eng = _engine(n_slots=1)
    sched = Scheduler(eng)
    p = _prompt(cfg, 16, 41)
    s = Sampling(temperature=0.9, top_k=20, top_p=0.95, seed=123, max_tokens=10)
    a = generate(sched, [p], s)[0]
    b = generate(sched, [p], s)[0]
    assert a == b and len(a) == 10
    lg = torch.randn(500, generator=torch.Generator().manual_seed(0))
    pr = dist(lg, Sampling(temperature=1.0, top_k=7))
    assert int((pr > 0).sum()) == 7 and abs(float(pr.sum()) - 1) < 1e-6
    pr = dist(lg, Sampling(temperature=1.0, top_p=0.5))
    sp = torch.sort(torch.softmax(lg, -1), descending=True).values
    k = int((torch.cumsum(sp, 0) < 0.5).sum()) + 1
    assert int((pr > 0).sum()) == k
    pr = dist(lg, Sampling(temperature=1.0, min_p=0.2))
    sm = torch.softmax(lg, -1)
    assert int((pr > 0).sum()) == int((sm >= 0.2 * sm.max()).sum())


def test_speculative_sampling_preserves_the_distribution():
    """Point-mass drafts accepted with probability p(draft), replaced from p \\ {draft} otherwise: first-token
    frequencies match the target distribution."""
    lg = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0]] * 2)
    want = torch.softmax(lg[0], -1)
    counts = torch.zeros(5)
    for seed in range(4000):
        s = Sampler(Sampling(temperature=1.0, seed=seed))
        counts[s.spec_accept(lg, [1])[0]] += 1
    assert torch.allclose(counts / counts.sum(), want, atol=0.03)


def test_stop_token_and_cancel_and_guard():
    cfg, w, eng = _engine(n_slots=1)
    p = _prompt(cfg, 10, 51)
    ref = _plain(cfg, w, p, 8)
    sched = Scheduler(eng)
    out = generate(sched, [p], Sampling(max_tokens=8, stop_ids=[ref[3]]))[0]
    assert out == ref[:ref.index(ref[3])]
    events = []
    req = Request(p, Sampling(max_tokens=50), events.append, guard=lambda toks: "guard" if len(events) >= 3 else None)
    sched.submit(req)
    while not any(e.kind == "finish" for e in events):
        sched.run_once()
    assert events[-1].reason == "guard"
    events2 = []
    req2 = Request(p, Sampling(max_tokens=50), events2.append)
    sched.submit(req2)
    sched.run_once(); sched.run_once()
    req2.cancel.set()
    while not any(e.kind == "finish" for e in events2):
        sched.run_once()
    assert events2[-1].reason == "cancelled" and sched.running == 0 and len(sched.free) == 1


def test_step_failures_kill_the_engine_after_three(monkeypatch):
    cfg, w, eng = _engine(n_slots=1)
    sched = Scheduler(eng)
    calls = {"n": 0}

    def boom(*a, **k):
        calls["n"] += 1
        raise RuntimeError("injected step failure")

    monkeypatch.setattr(eng, "forward", boom)
    died = False
    for i in range(3):
        evs = []
        sched.submit(Request(_prompt(cfg, 5, 60 + i), Sampling(max_tokens=3), evs.append))
        try:
            sched.run_once()
        except RuntimeError:
            died = True
            break
        assert evs and evs[-1].kind == "error"                   # the request fails, the engine keeps serving
    assert died and calls["n"] == 3


def test_pcache_structures():
    sc = SlotCache(tokens=list(range(50)))
    for p in (10, 20, 30, 40):
        sc.push(Snap(p, None, pinned=(p == 10)))
    assert [s.pos for s in sc.snaps] == [10, 30, 40]              # pinned first + KEEP_LAST 2
    assert sc.best_snap(list(range(35)) + [99]).pos == 30
    assert sc.best_snap(list(range(30))).pos == 10                # a snapshot at len(prompt) leaves nothing to run
    sc.truncate(30)
    assert [s.pos for s in sc.snaps] == [10, 30] and len(sc.tokens) == 30
    park = Park(4)
    park.add(list(range(100)), [Snap(64, None)], [1, 2])
    e, s = park.best(list(range(80)))
    assert s.pos == 64 and park.has_prefix(list(range(80)), 64) and not park.has_prefix([5, 6, 7], 1)
    assert common_prefix([1, 2, 3], [1, 2, 4]) == 2
    c = Copier()
    c.sync(list(range(30)) + list(range(10, 17)))
    assert c.propose(4) == [17, 18, 19, 20]
    r = SplitMix64(7)
    assert 0 <= r.uniform() < 1


def test_shared_prefill_forks_from_the_running_request():
    """Two requests with a long common prefix arriving together: the second waits until the first has passed the
    shared point, then forks its pages and state there instead of computing the prefix again; outputs are those of
    independent runs."""
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(21)
    base = torch.randint(0, cfg.vocab, (160,), generator=g).tolist()
    p1 = base + torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    p2 = base + torch.randint(0, cfg.vocab, (9,), generator=g).tolist()
    ecfg = EngineConfig(n_slots=2, max_ctx=512, prefill_chunk=64)
    want = [generate(Scheduler(Engine(cfg, w, ecfg, device="cpu"), SchedOptions()), [p], Sampling(max_tokens=8))[0]
            for p in (p1, p2)]
    sched = Scheduler(Engine(cfg, w, ecfg, device="cpu"), SchedOptions(share_min=64))
    got = generate(sched, [p1, p2], Sampling(max_tokens=8))
    assert got == want
    assert sched.stats.get("forked", 0) == 1
    assert sched.stats["cached_tokens"] >= 128


def test_mixed_steps_decode_rows_ride_with_prompt_chunks():
    # (decode_share=0 below: this test counts steps; the fairness rule, which inserts decode-only steps, has its own test)
    """A request that is decoding keeps producing tokens while another one prefills: both share forwards, and the
    tokens are those of separate runs."""
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(31)
    p1 = torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    p2 = torch.randint(0, cfg.vocab, (200,), generator=g).tolist()
    ecfg = EngineConfig(n_slots=2, max_ctx=512, prefill_chunk=64)
    want = [generate(Scheduler(Engine(cfg, w, ecfg, device="cpu"), SchedOptions(mixed=False)), [p], Sampling(max_tokens=12))[0]
            for p in (p1, p2)]
    sched = Scheduler(Engine(cfg, w, ecfg, device="cpu"), SchedOptions(mixed=True, decode_share=0.0))
    outs, done = [[], []], [False, False]

    def sink(i):
        def f(ev):
            if ev.kind == "tokens":
                outs[i].extend(ev.tokens)
            else:
                done[i] = True
        return f
    sched.submit(Request(list(p1), Sampling(max_tokens=12), sink(0)))
    for _ in range(2):                       # the first request reaches decoding
        sched.run_once()
    sched.submit(Request(list(p2), Sampling(max_tokens=12), sink(1)))
    steps_before = sched.stats["steps"]
    while not all(done):
        sched.run_once()
    assert outs == want
    # 200 prompt tokens in 64-row chunks = 4 chunk steps; without mixing the decode steps of request 1 would add to them
    assert sched.stats["steps"] - steps_before <= 4 + 12


def _mtp_setup(n_slots=1):
    from ferrite_b200.models.mtp import MtpDrafter
    cfg, w, eng = _engine(n_slots=n_slots)
    last = cfg.n_layers - 1
    for c in (cfg, eng.cfg, eng.ex.cfg, eng.full_cfg):
        c.tap_layers = [last]
    return cfg, w, eng, MtpDrafter(eng, n_slots=n_slots, max_ctx=256, depth=3)


def test_mtp_chain_drafter_keeps_greedy_output():
    cfg, w, eng, dr = _mtp_setup()
    sched = Scheduler(eng, SchedOptions(spec=3, copy_rows=False), drafter=dr)
    prompt = _prompt(cfg, 25, 31)
    out = generate(sched, [prompt], Sampling(max_tokens=14))[0]
    assert out == _plain(cfg, w, prompt, 14)
    assert sched.stats["drafted"] > 0
    assert dr.eng.ex.w["embed"].data_ptr() == eng.ex.w["embed"].data_ptr()       # the head shares the target's table


def test_mtp_rows_do_not_depend_on_how_the_prompt_was_cut():
    """The head's cache after absorbing a prompt in one piece or in two gives the same chain of drafts, and a draft
    run leaves no trace (drafting twice gives the same tokens)."""
    from ferrite_b200.engine.executor import Segment
    cfg, w, eng, dr = _mtp_setup()
    p = _prompt(cfg, 30, 5)
    eng.forward([Segment(0, 0, p, "none")])
    dr.absorb(0, p, 0, eng.taps)
    a = dr.draft(0, 9, 30, eng.taps, 3)
    assert len(a) == 3 and dr.draft(0, 9, 30, eng.taps, 3) == a
    eng.reset_slot(0); dr.reset(0)
    eng.forward([Segment(0, 0, p[:17], "none")])
    dr.absorb(0, p[:17], 0, eng.taps)
    eng.forward([Segment(0, 17, p[17:], "none")])
    dr.absorb(0, p[17:], 17, eng.taps)
    assert dr.draft(0, 9, 30, eng.taps, 3) == a
    assert dr.draft(0, 9, 29, eng.taps, 3) == []          # no hidden kept for that position: nothing to draft from


def test_group_prefill_runs_several_prompts_in_one_forward():
    cfg, w, eng = _engine(n_slots=4)
    prompts = [_prompt(cfg, n, 50 + n) for n in (40, 23, 64)]
    calls = []
    fwd = eng.forward

    def spy(segs, **kw):
        calls.append([len(s.tokens) for s in segs])
        return fwd(segs, **kw)
    eng.forward = spy
    sched = Scheduler(eng, SchedOptions(spec=0))
    out = generate(sched, prompts, Sampling(max_tokens=6))
    for p, o in zip(prompts, out):
        assert o == _plain(cfg, w, p, 6)
    assert len(calls[0]) == 3 and sum(calls[0]) >= 23 + 32 + 32      # all three prompts share the first forward
    # sampled requests take their first token from the logits of the shared forward
    s = Sampling(temperature=0.7, top_k=20, seed=3, max_tokens=5)
    a = generate(sched, prompts[:2], s)
    b = generate(sched, prompts[:2], s)
    assert a == b and all(len(x) == 5 for x in a)


def test_temperature_zero_with_penalties_does_not_depend_on_the_batch():
    """A temperature-0 request with penalties is not "greedy" for the device arg-max path: it gets the host sampler's
    penalised arg-max whether it runs alone or beside a sampled request (reference `greedy()`, `sched.rs:162`)."""
    s = Sampling(temperature=0.0, frequency_penalty=1.5, presence_penalty=0.5, max_tokens=14)
    assert s.argmax and not s.greedy and Sampling(temperature=0.0).greedy
    cfg, w, eng = _engine(n_slots=2)
    p = _prompt(cfg, 24, 31)
    alone = generate(Scheduler(eng), [p], s)[0]
    cfg, w, eng = _engine(n_slots=2)
    sched = Scheduler(eng)
    other = Sampling(temperature=0.9, top_k=20, seed=3, max_tokens=14)
    outs = generate(sched, [p, _prompt(cfg, 24, 32)], [s, other])
    assert outs[0] == alone
    assert alone != _plain(cfg, w, p, 14)                      # the penalties did change the output


def test_repetition_penalty_counts_the_prompt():
    logits = torch.zeros(16)
    logits[3], logits[5] = 4.0, 3.9
    s = Sampling(temperature=0.0, repetition_penalty=2.0)
    assert Sampler(s, prompt=[1, 2]).sample(logits) == 3
    assert Sampler(s, prompt=[3, 2]).sample(logits) == 5      # token 3 is in the prompt: 4.0 / 2 < 3.9
    smp = Sampler(Sampling(temperature=0.0, presence_penalty=1.0), prompt=[3])
    assert smp.sample(logits) == 3                            # presence / frequency look at generated tokens only
    smp.observe(3)
    assert smp.sample(logits) == 5


def test_decode_share_interleaves_decode_only_steps_with_prompt_chunks():
    """While a stream decodes and a long prompt is pending, prompt chunks are capped (`prefill_cap`) and decode-only steps
    are inserted until decoding has had its share of the (fake) wall time; the outputs stay the plain greedy ones."""
    cfg, w, eng = _engine(n_slots=2, max_ctx=512, chunk=64)
    sched = Scheduler(eng, SchedOptions(decode_share=0.5, prefill_cap=64, mixed=False, arrival_ms=0))
    now = [0.0]
    sched.clock = lambda: now[0]
    short, long_p = _prompt(cfg, 8, 41), _prompt(cfg, 200, 42)
    outs, done = [[], []], [False, False]

    def sink(i):
        def f(ev):
            if ev.kind == "tokens":
                outs[i].extend(ev.tokens)
            else:
                done[i] = True
        return f
    sched.submit(Request(short, Sampling(max_tokens=40), sink(0)))
    sched.run_once()                                   # the short prompt is in and decoding
    sched.submit(Request(long_p, Sampling(max_tokens=4), sink(1)))
    kinds = []
    orig_prefill = sched._group_prefill

    def prefill(prefills, budget):                     # a step with prompt rows costs 4 time units, a decode-only step 1
        n = orig_prefill(prefills, budget)
        now[0] += 3.0
        kinds.append(n)
        return n
    sched._group_prefill = prefill
    guard = 0
    while not all(done) and guard < 500:
        sched.run_once()
        now[0] += 1.0
        guard += 1
    assert all(done)
    assert outs[0] == _plain(cfg, w, short, 40) and outs[1] == _plain(cfg, w, long_p, 4)
    assert sched.stats.get("decode_only_steps", 0) >= 3          # decoding got steps of its own between the chunks
    assert kinds and max(kinds) <= 64 + 16                       # every prompt chunk respected the cap (a tail of <= 16 rows merges)


def test_arrival_window_collects_requests_sent_together():
    import threading
    import time as _time
    cfg, w, eng = _engine(n_slots=4)
    sched = Scheduler(eng, SchedOptions(arrival_ms=40, arrival_max_ms=400))
    prompts = [_prompt(cfg, 12, 50 + i) for i in range(3)]
    outs = [[] for _ in prompts]
    done = [threading.Event() for _ in prompts]

    def sink(i):
        def f(ev):
            if ev.kind == "tokens":
                outs[i].extend(ev.tokens)
            else:
                done[i].set()
        return f
    sched.start()
    try:
        for i, p in enumerate(prompts):              # sent 10 ms apart: inside the window
            sched.submit(Request(p, Sampling(max_tokens=3), sink(i)))
            _time.sleep(0.01)
        assert all(d.wait(30) for d in done)
    finally:
        sched.stop()
    # all three were admitted before the first step ran: one group prefill
    assert sched.stats["steps"] <= 1 + 3 + 1
    for p, o in zip(prompts, outs):
        assert o == _plain(cfg, w, p, 3)


def test_copier_adapts_its_length_continues_loops_and_grafts_onto_trees():
    from ferrite_b200.engine.copy import Copier, graft
    c = Copier(lo=4, hi=32)
    seq = list(range(100, 120)) + [7, 8, 9] + list(range(100, 110))          # the tail repeats the head
    c.sync(seq)
    assert c.propose(64, adaptive=True) == list(range(110, 114))              # starts at `lo` rows
    c.observe(4, 4)
    assert len(c.propose(64, adaptive=True)) == 8                             # a proposal that lands whole doubles
    c.observe(8, 8); c.observe(16, 16); c.observe(32, 32)
    assert c.extra == 32                                                      # ... up to `hi`
    c.observe(32, 10)
    assert c.extra == 16                                                      # less than half landed: halves
    assert c.propose(6) == list(range(110, 116))                              # the plain form proposes what is asked for
    for _ in range(4):
        c.observe(4, 0)
    assert c.propose(64) == [] and c.extra == 4                               # four misses: quiet, and back to `lo`
    # a loop of period 3 continues past the end of the history
    p = Copier()
    p.sync([1, 2, 3] * 4)
    assert p.propose(7) == [1, 2, 3, 1, 2, 3, 1]
    # graft: the copy 5 6 7 8 onto a tree root -> {5 -> {6, 9}, 4}
    toks, par = [0, 5, 4, 6, 9], [-1, 0, 0, 1, 1]
    followed, added = graft(toks, par, [5, 6, 7, 8], room=1)
    assert (followed, added) == (2, 1) and toks == [0, 5, 4, 6, 9, 7] and par == [-1, 0, 0, 1, 1, 3]
    toks, par = [0], [-1]
    assert graft(toks, par, [5, 6], room=8) == (0, 2) and par == [-1, 0, 1]


def test_block_drafter_window_bounds_its_context():
    """A drafter with a window keeps at most `ring` tokens in its own cache however long the sequence gets, is rebuilt
    from the last `window` committed tokens when a commit would run past the ring, and right after a rebuild drafts what
    a fresh drafter that saw exactly those tokens drafts. Greedy output through the scheduler stays the target's."""
    from ferrite_b200.models.drafter import BlockDrafter, drafter_config_for
    cfg, w, eng = _engine(n_slots=1)
    dcfg = drafter_config_for(cfg)
    hid = cfg.hidden
    mk = lambda **kw: BlockDrafter(dcfg, target_hidden=hid, n_taps=1, n_slots=1, max_ctx=512, device="cpu", block=4, **kw)
    win = mk(window=16, ring=40)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(1, cfg.vocab, (300,), generator=g).tolist()
    feats = torch.randn(300, hid, generator=g)
    pos, rebuilt_at = 0, []
    for n in [37, 5, 1, 1, 9, 1, 1, 30, 1, 1, 1, 60, 1, 1]:                # prompt chunks, decode rows, a long chunk
        base0 = win.base[0]
        win.absorb(0, toks[pos:pos + n], pos, [feats[pos:pos + n]])
        pos += n
        assert win.eng.slot_len[0] <= 40 and win.eng.slot_len[0] == pos - win.base[0]
        if win.base[0] != base0:
            rebuilt_at.append(pos)
    assert len(rebuilt_at) >= 3
    d_win = win.draft(0, toks[pos - 1], pos, None, 4)
    # a fresh, unbounded drafter fed exactly what the windowed one holds (same local positions) drafts the same
    held = pos - win.base[0]
    fresh = mk()
    fresh.absorb(0, toks[pos - held:pos], 0, [feats[pos - held:pos]])
    assert fresh.draft(0, toks[pos - 1], held, None, 4) == d_win and len(d_win) == 4
    # snapshot / restore: same base -> length rolls back; after a rebuild -> the slot starts over
    blob = win.save_window(0)
    win.absorb(0, toks[pos:pos + 2], pos, [feats[pos:pos + 2]])
    win.restore_window(0, blob)
    assert win.eng.slot_len[0] == blob["len"] and win._hist_tokens(0) <= 16
    win.absorb(0, toks[pos:pos + 30], pos, [feats[pos:pos + 30]])          # forces a rebuild
    win.restore_window(0, blob)
    assert win.eng.slot_len[0] == 0 and win.hist[0] == []
    # through the scheduler: speculation with a windowed drafter keeps the greedy text
    p = _prompt(cfg, 50, 21)
    cfg.tap_layers = [cfg.n_layers - 1]
    eng2 = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256), device="cpu")
    dr = BlockDrafter(dcfg, target_hidden=hid, n_taps=1, n_slots=1, max_ctx=256, device="cpu", block=4, window=16, ring=40)
    out = generate(Scheduler(eng2, SchedOptions(spec=3, copy_rows=False), drafter=dr), [p], Sampling(max_tokens=40))[0]
    assert out == _plain(cfg, w, p, 40) and dr.eng.slot_len[0] <= 40


def test_common_prefix_matches_the_token_by_token_loop():
    import random
    rng = random.Random(0)
    for _ in range(1500):
        n = rng.randrange(0, 500)
        a = [rng.randrange(3) for _ in range(n)]
        b = a[:rng.randrange(0, n + 1)] + [rng.randrange(3) for _ in range(rng.randrange(0, 40))]
        want = next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), min(len(a), len(b)))
        assert common_prefix(a, b) == want and common_prefix(tuple(a), b) == want


def test_end_of_reply_snapshot_in_a_verify_step_holds_the_committed_state():
    """A request that ends inside a speculative step snapshots its slot for the next turn: the snapshot must hold the
    recurrent state after the accepted rows were committed (it is labelled with that position), not the state the step
    started from."""
    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.sampler import Sampling
    from ferrite_b200.engine.scheduler import SchedOptions, Scheduler, generate
    from ferrite_b200.models.drafter import OracleDrafter
    cfg = tiny_hybrid()
    g = torch.Generator().manual_seed(1)
    p1 = torch.randint(1, cfg.vocab, (40,), generator=g).tolist()
    mk = lambda: Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=256, prefill_chunk=64), device="cpu")
    for n_out in (9, 12):
        out1 = mk().generate(p1, n_out)
        eng = mk()
        dr = OracleDrafter(1.0, cfg.vocab)
        dr.set_truth(0, len(p1), out1)
        sched = Scheduler(eng, SchedOptions(spec=4, arrival_ms=0), drafter=dr)
        assert generate(sched, [p1], Sampling(max_tokens=n_out))[0] == out1
        assert sched.stats["accepted"] > 0
        snap = sched.slot_cache[0].snaps[-1]
        assert snap.pos == len(p1) + n_out - 1
        ref = mk()
        ref.prefill(0, (p1 + out1)[:snap.pos])
        want = ref.ex.state_save(0)
        assert float((want["rec"] - snap.state["gdn"]["rec"]).abs().max()) < 1e-5
        assert float((want["conv"] - snap.state["gdn"]["conv"]).abs().max()) < 1e-5


def test_drafter_passes_are_batched_over_the_requests_of_a_step():
    """Three requests decoding together with a block drafter: the drafter runs one draft pass and one absorb pass per
    step for all of them (not one per request), drafts what the one-by-one path drafts, and the text stays the plain one.
    Chains and trees."""
    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.sampler import Sampling
    from ferrite_b200.engine.scheduler import Drafter, SchedOptions, Scheduler, generate
    from ferrite_b200.models.drafter import BlockDrafter, drafter_config_for
    cfg = tiny_hybrid()
    cfg.tap_layers = [0, 2]
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(1, cfg.vocab, (n,), generator=g).tolist() for n in (20, 33, 27)]
    mk = lambda: Engine(cfg, None, EngineConfig(n_slots=3, max_ctx=256, prefill_chunk=64), device="cpu")
    plain = generate(Scheduler(mk(), SchedOptions(spec=0, arrival_ms=0)), prompts, Sampling(max_tokens=14))
    for tree_rows in (0, 6):
        stats = []
        for batched in (True, False):
            dr = BlockDrafter(drafter_config_for(cfg), target_hidden=cfg.hidden, n_taps=2, n_slots=3, max_ctx=256,
                              device="cpu", block=6)
            if not batched:                           # the interface's defaults: one request at a time
                dr.draft_many = lambda reqs, taps, dr=dr: Drafter.draft_many(dr, reqs, taps)
                dr.draft_tree_many = lambda reqs, taps, dr=dr: Drafter.draft_tree_many(dr, reqs, taps)
                dr.absorb_rows_many = lambda items, taps, dr=dr: Drafter.absorb_rows_many(dr, items, taps)
            calls = {"n": 0}
            fwd = dr.eng.forward

            def counted(*a, _fwd=fwd, _c=calls, **kw):
                _c["n"] += 1
                return _fwd(*a, **kw)
            dr.eng.forward = counted
            sched = Scheduler(mk(), SchedOptions(spec=4, tree_rows=tree_rows, arrival_ms=0), drafter=dr)
            assert generate(sched, prompts, Sampling(max_tokens=14)) == plain
            stats.append((sched.stats["drafted"], sched.stats["accepted"], calls["n"]))
        (d1, a1, n1), (d0, a0, n0) = stats
        assert (d1, a1) == (d0, a0) and d1 > 0          # the same drafts either way
        assert n1 < 0.6 * n0, (n1, n0)                  # and far fewer passes of the draft model


def test_mtp_head_drafts_for_all_requests_of_a_step_in_one_pass_per_depth():
    from ferrite_b200.engine.scheduler import Drafter
    stats = []
    for batched in (True, False):
        cfg, w, eng, dr = _mtp_setup(n_slots=3)
        if not batched:
            dr.draft_many = lambda reqs, taps, dr=dr: Drafter.draft_many(dr, reqs, taps)
        calls = {"n": 0}
        fwd = dr.eng.forward

        def counted(*a, _fwd=fwd, _c=calls, **kw):
            _c["n"] += 1
            return _fwd(*a, **kw)
        dr.eng.forward = counted
        sched = Scheduler(eng, SchedOptions(spec=3, copy_rows=False, arrival_ms=0), drafter=dr)
        prompts = [_prompt(cfg, n, 70 + n) for n in (25, 31, 19)]
        out = generate(sched, prompts, Sampling(max_tokens=12))
        for p, o in zip(prompts, out):
            assert o == _plain(cfg, w, p, 12)
        stats.append((sched.stats["drafted"], sched.stats["accepted"], calls["n"]))
    assert stats[0][:2] == stats[1][:2] and stats[0][0] > 0
    assert stats[0][2] < stats[1][2]


@pytest.mark.parametrize("seed,kind", [(1, "tree"), (2, "block"), (4, "copy")])
def test_every_snapshot_holds_the_state_of_its_prefix(seed, kind):
    """Random multi-turn conversations under speculation (few slots, so conversations are parked and resumed): after every
    round each snapshot kept by a slot or by the park pool must hold exactly the recurrent state a fresh engine has after
    the snapshot's token prefix, the drafter window saved with it must end at the same position, and every reply must be
    the plain greedy one. Token equality alone does not catch a stale state on a small model; this does."""
    import random

    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.models.drafter import BlockDrafter, drafter_config_for
    cfg = tiny_hybrid()
    cfg.tap_layers = [0, 2]
    mk = lambda n: Engine(cfg, None, EngineConfig(n_slots=n, max_ctx=512, prefill_chunk=64), device="cpu")
    ref = mk(1)

    def state_at(tokens):
        ref.reset_slot(0)
        ref.prefill(0, tokens)
        return ref.ex.state_save(0)

    def check(holder, tokens, where):
        for sn in holder.snaps:
            if sn.pos > len(tokens):
                continue
            w = state_at(tokens[:sn.pos])
            for k in ("rec", "conv"):
                assert float((w[k] - sn.state["gdn"][k]).abs().max()) < 1e-4, (where, sn.pos, k)
            blob = sn.state.get("draft")
            # (a drafter that started over after a restore it could not follow counts its rows from `base`)
            assert blob is None or blob["base"] + blob["len"] == sn.pos, (where, sn.pos, blob["base"], blob["len"])

    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    eng = mk(rnd.choice([1, 2]))
    dr = None if kind == "copy" else BlockDrafter(drafter_config_for(cfg), target_hidden=cfg.hidden, n_taps=2,
                                                  n_slots=eng.ecfg.n_slots, max_ctx=512, device="cpu", block=6)
    sched = Scheduler(eng, SchedOptions(spec=rnd.choice([2, 4, 6]), tree_rows=6 if kind == "tree" else 0, arrival_ms=0), drafter=dr)
    convs = [torch.randint(1, cfg.vocab, (rnd.randint(20, 120),), generator=g).tolist() for _ in range(3)]
    for turn in range(4):
        ks = rnd.sample(range(3), rnd.choice([1, 2]))
        n_out = rnd.randint(3, 12)
        hints = [[64 * rnd.randint(1, max(1, len(convs[i]) // 64))] if len(convs[i]) > 64 else [] for i in ks]
        outs = generate(sched, [convs[i] for i in ks], Sampling(max_tokens=n_out), snapshots=hints)
        for i, o in zip(ks, outs):
            ref.reset_slot(0)
            assert o == ref.generate(convs[i], n_out, slot=0), (turn, i)
            convs[i] = convs[i] + o + torch.randint(1, cfg.vocab, (rnd.randint(1, 9),), generator=g).tolist()
        for slot, sc in enumerate(sched.slot_cache):
            check(sc, sc.tokens, f"slot {slot} turn {turn}")
        for key, e in sched.park.entries.items():
            check(e, e.tokens, f"park {key} turn {turn}")
    assert sched.stats["cached_tokens"] > 0 and sched.stats["accepted"] > 0


def test_stop_token_inside_a_verify_step_leaves_a_resumable_slot():
    """The stop token is accepted in the middle of a verify step: the rows behind it are not committed, the reply ends
    there, and the next turn (reply + stop token + new text) resumes from the end-of-reply snapshot with the true state."""
    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.models.drafter import OracleDrafter
    cfg = tiny_hybrid()
    mk = lambda: Engine(cfg, None, EngineConfig(n_slots=1, max_ctx=512, prefill_chunk=64), device="cpu")
    ref = mk()
    hits = 0
    for seed in range(40):
        g = torch.Generator().manual_seed(300 + seed)
        p = torch.randint(1, cfg.vocab, (30,), generator=g).tolist()
        ref.reset_slot(0)
        plain = ref.generate(p, 12, slot=0)
        j = next((i for i in range(2, 9) if plain[i] not in plain[:i]), None)   # a stop token first seen mid-reply
        if j is None:
            continue
        hits += 1
        eng = mk()
        dr = OracleDrafter(1.0, cfg.vocab)
        dr.set_truth(0, len(p), plain)
        sched = Scheduler(eng, SchedOptions(spec=6, arrival_ms=0), drafter=dr)
        out = generate(sched, [p], Sampling(max_tokens=12, stop_ids=[plain[j]]))[0]
        assert out == plain[:j]
        assert eng.slot_len[0] == len(p) + j                  # nothing behind the reply was committed
        snap = sched.slot_cache[0].snaps[-1]
        assert snap.pos == len(p) + j
        ref.reset_slot(0)
        ref.prefill(0, (p + plain)[:snap.pos])
        want = ref.ex.state_save(0)
        assert float((want["rec"] - snap.state["gdn"]["rec"]).abs().max()) < 1e-5
        p2 = p + out + [plain[j]] + torch.randint(1, cfg.vocab, (5,), generator=g).tolist()
        ref.reset_slot(0)
        want2 = ref.generate(p2, 5, slot=0)
        dr.truth.clear()
        before = sched.stats["cached_tokens"]
        assert generate(sched, [p2], Sampling(max_tokens=5))[0] == want2
        assert sched.stats["cached_tokens"] - before == len(p) + j
        if hits >= 3:
            break
    assert hits >= 1


@pytest.mark.parametrize("seed", [3, 4])
def test_kv_pages_are_never_lost_or_held_twice(seed):
    """Random multi-turn traffic over few slots and a small page pool (conversations are parked, resumed, evicted): after
    every round each KV page is in exactly one place: a slot's table, a parked entry, or the free list."""
    import random

    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    cfg = tiny_hybrid()
    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(900 + seed)
    eng = Engine(cfg, None, EngineConfig(n_slots=rnd.choice([1, 2, 3]), max_ctx=1024, prefill_chunk=64,
                                         kv_block=rnd.choice([16, 64])), device="cpu")
    sched = Scheduler(eng, SchedOptions(spec=rnd.choice([0, 4]), arrival_ms=0))
    convs = [torch.randint(1, cfg.vocab, (rnd.randint(20, 200),), generator=g).tolist() for _ in range(5)]
    for turn in range(6):
        ks = rnd.sample(range(5), rnd.choice([1, 2, 3]))
        outs = generate(sched, [convs[i] for i in ks], Sampling(max_tokens=rnd.randint(2, 10)))
        for i, o in zip(ks, outs):
            convs[i] = convs[i] + o + torch.randint(1, cfg.vocab, (rnd.randint(1, 30),), generator=g).tolist()
            if len(convs[i]) > 800:
                convs[i] = convs[i][:100]
        pool = eng.ex.pool
        held = [b for s in eng.ex.slot_blocks for b in s] + [b for e in sched.park.entries.values() for b in e.blocks]
        pages = held + list(pool.free)
        assert len(pages) == len(set(pages)) == pool.n_blocks, (turn, len(pages), len(set(pages)), pool.n_blocks)


def test_drafter_window_is_not_rolled_back_onto_another_conversations_rows():
    """A window snapshot names rows of the drafter's cache. Restored into a slot that holds other tokens at those rows
    (another conversation used it, or it is another slot), the drafter must start over instead of drafting from foreign
    rows; restored into the slot that still holds them, only the length rolls back."""
    import torch

    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment
    from ferrite_b200.models.drafter import BlockDrafter, drafter_config_for
    cfg = tiny_hybrid()
    cfg.tap_layers = [0, 2]
    eng = Engine(cfg, None, EngineConfig(n_slots=2, max_ctx=256, prefill_chunk=64), device="cpu")
    dr = BlockDrafter(drafter_config_for(cfg), target_hidden=cfg.hidden, n_taps=2, n_slots=2, max_ctx=256, device="cpu", block=6)
    g = torch.Generator().manual_seed(8)
    a = torch.randint(1, cfg.vocab, (60,), generator=g).tolist()
    b = torch.randint(1, cfg.vocab, (60,), generator=g).tolist()

    def feed(slot, toks, lo, hi):
        eng.forward([Segment(slot, lo, toks[lo:hi], "none")], commit=True)
        dr.absorb(slot, toks[lo:hi], lo, eng.taps)
    feed(0, a, 0, 40)
    blob = dr.save_window(0)
    want = dr.draft(0, a[40], 40, eng.taps, 6)
    feed(0, a, 40, 60)
    dr.restore_window(0, blob)                                  # same slot, same rows: a rollback
    assert dr.eng.slot_len[0] == 40 and dr.draft(0, a[40], 40, eng.taps, 6) == want
    # another conversation takes the slot, then the first one's snapshot comes back
    eng.reset_slot(0)
    dr.reset(0)
    feed(0, b, 0, 50)
    dr.restore_window(0, blob)
    assert dr.eng.slot_len[0] == 0 and dr.last_feat[0] is None      # started over: conversation b's rows are not a's
    # and into the other slot, which never held them
    feed(1, b, 0, 45)
    dr.restore_window(1, blob)
    assert dr.eng.slot_len[1] == 0
    # a drafter that started over works from the next absorbed row on, in its own positions
    eng.reset_slot(1)
    eng.forward([Segment(1, 0, a[:40], "none")], commit=True)
    feed(1, a, 40, 52)
    assert dr.base[1] == 40 and dr.eng.slot_len[1] == 12
    assert len(dr.draft(1, a[52], 52, eng.taps, 6)) == 6
