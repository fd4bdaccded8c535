"""The C++ host runtime (`csrc/host_runtime.cpp`) against the plain-Python statements of the same behaviour: copy
proposals, verify-tree walk / growth / grafting and the stop scanner must agree result for result on random cases."""
import random

import pytest
import torch

from ferrite_b200 import _ext

H = _ext.host()
pytestmark = pytest.mark.skipif(H is None, reason="extension not built")


def test_copy_index_matches_python(monkeypatch):
    from ferrite_b200.engine.copy import Copier
    rng = random.Random(1)
    for case in range(30):
        vocab = rng.choice([3, 8, 50])
        seq = [rng.randrange(vocab) for _ in range(rng.randrange(4, 400))]
        if case % 3 == 0:                                   # repeated spans, as in code edits
            seq = seq + seq[len(seq) // 3:] + seq[:20]
        nat = Copier()
        assert nat.native is not None
        monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
        ref = Copier()
        monkeypatch.delenv("FERRITE_NO_NATIVE_HOST")
        assert ref.native is None
        cut = rng.randrange(1, len(seq))
        for upto in (cut, len(seq), max(2, cut // 2), len(seq)):      # grow, grow, roll back, grow again
            part = seq[:upto] if upto >= cut else seq[:upto] + [vocab + 1]
            nat.sync(part)
            ref.sync(part)
            for want in (64, 7, 1):
                assert nat.propose(want) == ref.propose(want), (case, upto, want)
            nat.extra = ref.extra = rng.choice([4, 16])
            assert nat.propose(64, adaptive=True) == ref.propose(64, adaptive=True)


def test_tree_walk_grow_and_graft_match_python(monkeypatch):
    from ferrite_b200.engine import scheduler as S
    from ferrite_b200.engine.copy import graft
    rng = random.Random(2)
    for case in range(40):
        depth, width = rng.randrange(1, 7), rng.randrange(1, 5)
        cands = [sorted(((rng.randrange(20), -rng.random() * 3) for _ in range(rng.randrange(1, width + 1))),
                        key=lambda x: -x[1]) for _ in range(depth)]
        if case % 5 == 0:
            cands[0][0] = (cands[0][0][0], cands[0][-1][1])            # equal scores: the tie order must agree too
        rows = rng.randrange(1, 24)
        nat = S.grow_tree(cands, rows)
        monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
        ref = S.grow_tree(cands, rows)
        monkeypatch.delenv("FERRITE_NO_NATIVE_HOST")
        assert nat == ref, case
        toks, par = [5] + nat[0], [-1] + nat[1]
        target = [rng.choice(toks + [99]) for _ in toks]
        a = S.tree_walk(toks, par, list(target))
        b = S.tree_walk(toks, par, lambda node: target[node])          # the callable form is the Python walk
        assert a == b and a[0][0] == 0 and len(a[0]) == len(a[1])
        copy = [rng.choice(toks) for _ in range(rng.randrange(0, 6))]
        t1, p1 = list(toks), list(par)
        r1 = graft(t1, p1, copy, 3)
        monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
        t2, p2 = list(toks), list(par)
        r2 = graft(t2, p2, copy, 3)
        monkeypatch.delenv("FERRITE_NO_NATIVE_HOST")
        assert (r1, t1, p1) == (r2, t2, p2)


def test_stop_scanner_matches_python(monkeypatch):
    from ferrite_b200.server.stop import StopMatcher
    rng = random.Random(3)
    alphabet = ["a", "b", "<", "/", ">", "é", "日", "\n", "END"]
    for case in range(60):
        stops = ["".join(rng.choice(alphabet) for _ in range(rng.randrange(1, 5))) for _ in range(rng.randrange(1, 4))]
        text = "".join(rng.choice(alphabet) for _ in range(rng.randrange(0, 60)))
        if case % 2:
            at = rng.randrange(0, len(text) + 1)
            text = text[:at] + rng.choice(stops) + text[at:]
        include = bool(case % 3 == 0)
        nat = StopMatcher(stops, include)
        assert nat.native is not None
        monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
        ref = StopMatcher(stops, include)
        monkeypatch.delenv("FERRITE_NO_NATIVE_HOST")
        assert ref.native is None
        i = 0
        while i < len(text):
            n = rng.randrange(1, 6)
            assert nat.push(text[i:i + n]) == ref.push(text[i:i + n]), (case, stops, text, i)
            i += n
        assert nat.hit == ref.hit and nat.flush() == ref.flush()


def test_step_metadata_block_matches_python(monkeypatch):
    """`Executor._upload` through the C++ fill and through the Python loop: the staging block, the tree block and the
    logit rows are identical, for plain segments and for verify trees."""
    import torch
    from ferrite_b200.config import EngineConfig, tiny_hybrid
    from ferrite_b200.engine.engine import Engine
    from ferrite_b200.engine.executor import Segment, StepBatch
    eng = Engine(tiny_hybrid(), None, EngineConfig(n_slots=3, max_ctx=256), device="cpu")
    ex = eng.ex
    plain = StepBatch([Segment(0, 5, [11, 12, 13], "all"), Segment(2, 0, [7], "last"), Segment(1, 40, [1, 2], "none")], commit=True)
    tree = StepBatch([Segment(0, 9, [3, 4, 5, 6, 7], "all", parents=[-1, 0, 0, 1, 2]), Segment(1, 2, [8, 9], "all")], commit=False)
    for batch in (plain, tree):
        outs = []
        for native in (True, False):
            if native:
                monkeypatch.delenv("FERRITE_NO_NATIVE_HOST", raising=False)
            else:
                monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
            for buf in ex._ring + ex._tring:
                buf.zero_()
            ex._ring_i = 0
            rows = ex._upload(batch)
            T, S = batch.n_rows, len(batch.segments)
            outs.append((rows, ex._ring[0][:5 * T + 4 * S].clone(), ex._tring[0].clone() if batch.tree else None))
        (r1, h1, t1), (r2, h2, t2) = outs
        nl = len(r1)
        T = batch.n_rows
        assert r1 == r2 and torch.equal(h1[:4 * T + nl], h2[:4 * T + nl]) and torch.equal(h1[5 * T:], h2[5 * T:])
        if batch.tree:
            R = ex._R
            for blk in range(6):
                assert torch.equal(t1[blk * R:blk * R + (2 * T if blk == 0 else T)], t2[blk * R:blk * R + (2 * T if blk == 0 else T)]), blk


def test_native_sampler_matches_the_python_statements(monkeypatch):
    """The C++ sampler against the PyTorch statements of `engine/sampler.py`: the same support and probabilities over
    peaked and flat rows under every filter, the same draws for the same uniforms (boundary cases aside), the draft
    acceptance walk token for token on a seeded run, and a large-vocabulary row several times faster."""
    import time

    from ferrite_b200 import _ext
    from ferrite_b200.engine import sampler as S
    h = _ext.host()
    if h is None or not hasattr(h, "sample_probs"):
        pytest.skip("extension not built")
    g = torch.Generator().manual_seed(0)
    settings = [S.Sampling(temperature=0.8), S.Sampling(temperature=1.0, top_k=20), S.Sampling(temperature=0.7, top_p=0.9),
                S.Sampling(temperature=1.3, top_k=50, top_p=0.8, min_p=0.05), S.Sampling(temperature=1.0, min_p=0.2),
                S.Sampling(temperature=0.6, top_p=0.3)]
    same_draws = total_draws = 0
    for scale in (0.5, 3.0, 12.0):                      # flat, ordinary and peaked rows
        for s in settings:
            logits = torch.randn(5000, generator=g) * scale
            banned = [int(logits.argmax())] if s.top_k else []
            monkeypatch.delenv("FERRITE_NO_NATIVE_HOST", raising=False)
            got = S.dist(logits, s, banned)
            monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
            want = S.dist(logits, s, banned)
            assert torch.equal(got > 0, want > 0), (scale, s)
            assert torch.allclose(got, want, atol=1e-6, rtol=1e-4)
            assert abs(float(got.sum()) - 1.0) < 1e-5
            for k in range(50):
                seed = 1000 * k + 7
                monkeypatch.delenv("FERRITE_NO_NATIVE_HOST", raising=False)
                a = S.draw(got, S.SplitMix64(seed))
                a_ex = S.draw_excluding(got, S.SplitMix64(seed), int(got.argmax()))
                monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
                b = S.draw(want, S.SplitMix64(seed))
                b_ex = S.draw_excluding(want, S.SplitMix64(seed), int(want.argmax()))
                assert float(got[a]) > 0 and a_ex != int(got.argmax()) or float(got.max()) == 1.0
                same_draws += int(a == b) + int(a_ex == b_ex)
                total_draws += 2
    assert same_draws >= 0.995 * total_draws, (same_draws, total_draws)
    # a point mass: nothing else to draw, the excluded token comes back and the generator does not advance
    one = torch.zeros(100)
    one[17] = 1.0
    monkeypatch.delenv("FERRITE_NO_NATIVE_HOST", raising=False)
    rng = S.SplitMix64(5)
    assert S.draw_excluding(one, rng, 17) == 17 and rng.s == 5
    assert S.draw(one, rng) == 17
    # the acceptance walk over drafts, seeded: native and Python walk the same tokens
    logits_rows = torch.randn(5, 3000, generator=g) * 4
    drafts = [int(logits_rows[i].argmax()) for i in range(4)]
    outs = []
    for native in (True, False):
        if native:
            monkeypatch.delenv("FERRITE_NO_NATIVE_HOST", raising=False)
        else:
            monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
        smp = S.Sampler(S.Sampling(temperature=0.9, top_p=0.95, seed=11, presence_penalty=0.3))
        outs.append(smp.spec_accept(logits_rows, drafts))
    assert outs[0] == outs[1] and len(outs[0]) >= 1
    # cost on a vocabulary-sized peaked row
    big = torch.randn(248320, generator=g) * 6
    s = S.Sampling(temperature=0.8, top_k=0, top_p=0.9)
    times = []
    for native in (True, False):
        if native:
            monkeypatch.delenv("FERRITE_NO_NATIVE_HOST", raising=False)
        else:
            monkeypatch.setenv("FERRITE_NO_NATIVE_HOST", "1")
        S.draw(S.dist(big, s), S.SplitMix64(1))
        t0 = time.perf_counter()
        for k in range(5):
            S.draw(S.dist(big, s), S.SplitMix64(k))
        times.append((time.perf_counter() - t0) / 5)
    print(f"host sampler, 248K row, top-p: native {times[0] * 1e3:.2f} ms, PyTorch statements {times[1] * 1e3:.2f} ms")
    assert times[0] < times[1]


def test_repetition_mask_equals_the_set_union():
    """The sampler's incremental mask of prompt and generated ids gives the logits of the set-union statement."""
    from ferrite_b200.engine import sampler as S
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, 500, (300,), generator=g).tolist()
    s = S.Sampling(temperature=0.0, repetition_penalty=1.3, presence_penalty=0.2, frequency_penalty=0.1)
    smp = S.Sampler(s, prompt=prompt)
    for step in range(20):
        logits = torch.randn(500, generator=g) * 3
        want = S.penalize(logits.float(), smp.counts, s, smp.seen)
        got = smp._penalized(logits)
        assert torch.equal(got, want), step
        smp.observe(int(torch.randint(0, 500, (1,), generator=g)))
