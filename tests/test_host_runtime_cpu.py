"""The C++ host runtime (`csrc/host_runtime.cpp`) against the plain-Python statements of the same behaviour: copy
proposals, verify-tree walk / growth / grafting and the stop scanner must agree result for result on random cases."""
import random

import pytest

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
