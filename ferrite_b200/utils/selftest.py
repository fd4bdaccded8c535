"""Self-tests that run the engine against itself on any device (`python -m ferrite_b200.utils.selftest [tree]`).

Counterpart of the reference's `ferrite tree-test` / `selftest` commands (`crates/fe-cli/src/main.rs`,
`crates/fe-model/src/selftest.rs`: tree attention against one-row decode, tree GDN): here the check is end to end,
a verify tree against the chain verify of each of its root-to-node paths, then a committed path against a slot that was
fed the same tokens one after another.
"""
from __future__ import annotations

import sys
from typing import Optional

import torch

from ..config import EngineConfig, ModelConfig, tiny_hybrid
from ..engine.engine import Engine
from ..engine.executor import Segment
from ..models.weights import init_weights


def _paths(parents):
    """Every root-to-node path of the tree, as lists of row indices."""
    out = []
    for r in range(len(parents)):
        path, i = [], r
        while i >= 0:
            path.append(i)
            i = parents[i]
        out.append(path[::-1])
    return out


def tree_test(device: str = "cpu", tol: float = 2e-4, cfg: Optional[ModelConfig] = None, n_prompt: int = 37,
              kv_dtype: str = "bf16") -> float:
    """Returns the largest logit error seen (relative to the largest logit); raises AssertionError past `tol`."""
    cfg = cfg or tiny_hybrid()
    w = init_weights(cfg, seed=0) if cfg.hidden <= 512 else None
    mk = lambda: Engine(cfg, w, EngineConfig(n_slots=2, max_ctx=256, kv_dtype=kv_dtype), device=device, seed=0)  # noqa: E731
    tree, chain = mk(), mk()
    g = torch.Generator().manual_seed(1)
    p = torch.randint(0, cfg.vocab, (n_prompt,), generator=g).tolist()
    toks = torch.randint(0, cfg.vocab, (7,), generator=g).tolist()
    par = [-1, 0, 0, 1, 2, 3, 2]                   # leaves: 0-1-3-5, 0-2-4, 0-2-6
    for e in (tree, chain):
        e.forward([Segment(0, 0, p, "none")])
    got = tree.forward([Segment(0, n_prompt, toks, "all", parents=par)], commit=False, greedy=False)[0].clone()
    worst = 0.0
    for path in _paths(par):
        if len(path) < 2 and path != [0]:
            continue
        want = chain.forward([Segment(0, n_prompt, [toks[r] for r in path], "all")], commit=False, greedy=False)[0].clone()
        scale = max(1.0, want.abs().max().item())
        for j, r in enumerate(path):
            err = (got[r] - want[j]).abs().max().item() / scale
            worst = max(worst, err)
            assert err < tol, f"tree row {r} on path {path}: {err}"
    keep = [0, 2, 6]
    tree.commit_tree([keep])
    assert tree.slot_len[0] == n_prompt + len(keep)
    chain.forward([Segment(0, n_prompt, [toks[r] for r in keep], "none")])
    a = tree.forward([Segment(0, n_prompt + 3, [21], "last")], greedy=False)[0].clone()
    b = chain.forward([Segment(0, n_prompt + 3, [21], "last")], greedy=False)[0].clone()
    err = (a - b).abs().max().item() / max(1.0, b.abs().max().item())
    assert err < tol, f"decode after commit_tree: {err}"
    tree.check()
    return max(worst, err)


def main(argv) -> int:
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    what = argv[1] if len(argv) > 1 else "tree"
    if what == "tree":
        print(f"tree-test on {dev}: max relative logit error {tree_test(dev, 2e-4 if dev == 'cpu' else 3e-2):.3g}")
        return 0
    print(f"unknown self-test {what!r}; known: tree")
    return 2


if __name__ == "__main__":
    sys.exit(main(sys.argv))
