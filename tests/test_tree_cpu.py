"""Verify trees on the CPU ops: a tree step scores every root-to-node path as the chain verify of that path would, and
committing one path leaves the slot as if its tokens had been fed one by one."""
import pytest
import torch

from ferrite_b200.config import EngineConfig, tiny_hybrid
from ferrite_b200.engine.engine import Engine
from ferrite_b200.engine.executor import Segment, tree_layout
from ferrite_b200.models.weights import init_weights


def _prompt(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_tree_layout():
    #        0
    #      1   2
    #      3   4
    #      5
    depth, mask, flags = tree_layout([-1, 0, 0, 1, 2, 3])
    assert depth == [0, 1, 1, 2, 2, 3]
    assert mask == [0b1, 0b11, 0b101, 0b1011, 0b10101, 0b101011]
    assert flags[0] == 2 and flags[1] == 2 and flags[2] == 1 | 2 and flags[3] == 1 | 2 and flags[4] == 1 and flags[5] == 1
    with pytest.raises(AssertionError):
        tree_layout([-1, 2, 0])


def _engines(device="cpu", n=2, seed=0):
    cfg = tiny_hybrid()
    w = init_weights(cfg, seed=seed)
    return cfg, [Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256), device=device) for _ in range(n)]


def test_tree_verify_matches_chain_verify_cpu():
    from ferrite_b200.utils.selftest import tree_test
    assert tree_test("cpu", 2e-4) < 2e-4


def test_two_trees_and_a_chain_in_one_step_cpu():
    cfg, (tree, chain) = _engines("cpu")
    pa, pb = _prompt(cfg, 20, 3), _prompt(cfg, 33, 4)
    for e in (tree, chain):
        e.forward([Segment(0, 0, pa, "none")])
        e.forward([Segment(1, 0, pb, "none")])
    ta, para = [1, 2, 3, 4], [-1, 0, 0, 2]
    tb = [9, 8, 7]
    got = tree.forward([Segment(0, 20, ta, "all", parents=para), Segment(1, 33, tb, "all")], commit=False,
                       greedy=False)[0].clone()
    wa = chain.forward([Segment(0, 20, [1, 3, 4], "all")], commit=False, greedy=False)[0].clone()
    wb = chain.forward([Segment(1, 33, tb, "all")], commit=False, greedy=False)[0].clone()
    assert (got[[0, 2, 3]] - wa).abs().max().item() < 2e-4
    assert (got[4:] - wb).abs().max().item() < 2e-4
    tree.commit_tree([[0, 2], [0, 1, 2]])
    assert tree.slot_len == [22, 36]
    chain.forward([Segment(0, 20, [1, 3], "none"), Segment(1, 33, tb, "none")])
    a = tree.forward([Segment(0, 22, [6], "last"), Segment(1, 36, [6], "last")], greedy=False)[0].clone()
    b = chain.forward([Segment(0, 22, [6], "last"), Segment(1, 36, [6], "last")], greedy=False)[0].clone()
    assert (a - b).abs().max().item() < 2e-4


def test_grow_tree_and_walk():
    from ferrite_b200.engine.scheduler import grow_tree, tree_walk
    import math
    lp = math.log
    cands = [[(10, lp(0.6)), (11, lp(0.3)), (12, lp(0.1))], [(20, lp(0.5)), (21, lp(0.4))], [(30, lp(0.9))]]
    toks, par = grow_tree(cands, 6)
    assert len(toks) == 6 and par[0] == 0 and all(p <= i for i, p in enumerate(par))       # parents precede children
    # best path first: 10 (0.6), then 10-20 (0.30) ties 11 (0.30): both in, then 10-20-30 (0.27), 10-21 (0.24), 10-21-30 (0.216)
    paths = set()
    for i in range(6):
        seq, r = [], i + 1
        while r > 0:
            seq.append(toks[r - 1]); r = par[r - 1]
        paths.add(tuple(seq[::-1]))
    assert paths == {(10,), (11,), (10, 20), (10, 20, 30), (10, 21), (10, 21, 30)}
    # chain budget 1 keeps only the best token
    assert grow_tree(cands, 1) == ([10], [0])
    seg_toks, seg_par = [7] + toks, [-1] + par
    target = {(): 10, (10,): 21, (10, 21): 99}
    def pick(node):
        seq, r = [], node
        while r > 0:
            seq.append(seg_toks[r]); r = seg_par[r]
        return target[tuple(seq[::-1])]
    path, new = tree_walk(seg_toks, seg_par, pick)
    assert [seg_toks[r] for r in path] == [7, 10, 21] and new == [10, 21, 99]


def test_scheduler_tree_speculation_keeps_greedy_output():
    from ferrite_b200.config import ModelConfig
    from ferrite_b200.engine.scheduler import Sampling, SchedOptions, Scheduler, generate
    from ferrite_b200.models.drafter import BlockDrafter
    cfg = tiny_hybrid()
    cfg.tap_layers = [1, 3]
    w = init_weights(cfg, seed=0)
    prompt = _prompt(cfg, 25, 31)
    plain = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256), device="cpu")
    want = generate(Scheduler(plain, SchedOptions(spec=0)), [prompt, prompt[:11]], Sampling(max_tokens=14))
    eng = Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256), device="cpu")
    dcfg = ModelConfig(name="tiny-drafter", hidden=128, inter=256, n_layers=2, full_attn_every=1, head_dim=32, n_q=4,
                       n_kv=2, rotary_dim=32, attn_gate=False, vocab=cfg.vocab, tie_embeddings=True)
    dr = BlockDrafter(dcfg, target_hidden=cfg.hidden, n_taps=2, n_slots=2, max_ctx=256, device="cpu", block=4)
    sched = Scheduler(eng, SchedOptions(spec=4, copy_rows=False, tree_rows=10), drafter=dr)
    got = generate(sched, [prompt, prompt[:11]], Sampling(max_tokens=14))
    assert got == want
    assert sched.stats["drafted"] > 0
    # sampled requests walk the tree by sampling from the target at every node: seeded runs repeat
    s = Sampling(temperature=0.8, top_k=30, seed=5, max_tokens=10)
    a = generate(sched, [prompt], s)[0]
    b = generate(sched, [prompt], s)[0]
    assert a == b and len(a) == 10


def test_copy_rows_grafted_onto_the_draft_tree_keep_greedy_output():
    """A prompt made of repeated spans: the copy proposal is grafted onto the draft model's tree (shared rows followed, the
    rest hung below them); the text stays the plain greedy text and copy rows are among the drafts."""
    from ferrite_b200.config import ModelConfig
    from ferrite_b200.engine.scheduler import Sampling, SchedOptions, Scheduler, generate
    from ferrite_b200.models.drafter import BlockDrafter
    cfg = tiny_hybrid()
    cfg.tap_layers = [1, 3]
    w = init_weights(cfg, seed=0)
    prompt = _prompt(cfg, 12, 21) * 5
    plain = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256), device="cpu")
    want = generate(Scheduler(plain, SchedOptions(spec=0)), [prompt], Sampling(max_tokens=16))
    eng = Engine(cfg, w, EngineConfig(n_slots=1, max_ctx=256), device="cpu")
    dcfg = ModelConfig(name="tiny-drafter", hidden=128, inter=256, n_layers=2, full_attn_every=1, head_dim=32, n_q=4,
                       n_kv=2, rotary_dim=32, attn_gate=False, vocab=cfg.vocab, tie_embeddings=True)
    dr = BlockDrafter(dcfg, target_hidden=cfg.hidden, n_taps=2, n_slots=1, max_ctx=256, device="cpu", block=4)
    sched = Scheduler(eng, SchedOptions(spec=8, copy_rows=True, tree_rows=8), drafter=dr)
    got = generate(sched, [prompt], Sampling(max_tokens=16))
    assert got == want
    assert sched.stats["drafted"] > 0
