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
