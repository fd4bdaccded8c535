"""Score logits dumps against a stored top-k reference: the two-step KL workflow for checkpoints whose 16-bit run is too
big (or too slow) to keep next to every engine under test.

    python -m ferrite_b200.cli logits --model DIR --weights bf16 --ids-file seq.txt --out ref_logits.pt
    python -m ferrite_b200.utils.kl_score make-ref --logits ref_logits.pt --topk 64 --out ref_topk.pt
    python -m ferrite_b200.cli logits --model DIR --weights nvfp4 --ids-file seq.txt --out test_logits.pt
    python -m ferrite_b200.utils.kl_score score --ref ref_topk.pt --logits test_logits.pt [--skip 1024]

`make-ref` keeps, per position, the reference's `topk` largest log-probabilities, their token ids and the log of the mass
outside them. `score` computes per position KL(ref || test) over those k tokens plus one bucket for everything else
(a lower bound of the full KL that is tight once k covers the reference's mass), skips the first `--skip` positions
(the reference's method: a 1024-token prompt, then the teacher-forced rows are scored), and prints mean / max / per-file
figures as one JSON line; several `--logits` files give a per-sequence table. The role of the reference's `tools/kl.sh` +
`tools/kl_perseq.py`.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List

import torch


def make_ref(logits: torch.Tensor, topk: int) -> Dict[str, torch.Tensor]:
    lp = torch.log_softmax(logits.float(), -1)
    k = min(topk, lp.shape[-1])
    vals, ids = torch.topk(lp, k, dim=-1)
    rest = (1.0 - vals.exp().sum(-1)).clamp_min(1e-12).log()
    return {"logp": vals.to(torch.float32), "ids": ids.to(torch.int32), "rest": rest.to(torch.float32)}


def score(ref: Dict[str, torch.Tensor], logits: torch.Tensor, skip: int = 0) -> torch.Tensor:
    """Per-position KL(ref || test) in nats over the reference's top-k tokens and the remaining mass."""
    lq_full = torch.log_softmax(logits.float(), -1)
    n = min(lq_full.shape[0], ref["logp"].shape[0])
    lp, ids, rest = ref["logp"][:n], ref["ids"][:n].long(), ref["rest"][:n]
    lq = lq_full[:n].gather(-1, ids)
    q_rest = (1.0 - lq.exp().sum(-1)).clamp_min(1e-12).log()
    kl = (lp.exp() * (lp - lq)).sum(-1) + rest.exp() * (rest - q_rest)
    return kl[skip:]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("make-ref")
    p.add_argument("--logits", required=True)
    p.add_argument("--topk", type=int, default=64)
    p.add_argument("--out", required=True)
    p = sub.add_parser("score")
    p.add_argument("--ref", required=True)
    p.add_argument("--logits", required=True, nargs="+")
    p.add_argument("--skip", type=int, default=0)
    a = ap.parse_args(argv)
    if a.cmd == "make-ref":
        d = torch.load(a.logits)
        ref = make_ref(d["logits"], a.topk)
        ref["ids_in"] = torch.tensor(d.get("ids", []), dtype=torch.int64)
        torch.save(ref, a.out)
        mass = float(ref["logp"].exp().sum(-1).mean())
        print(json.dumps({"positions": int(ref["logp"].shape[0]), "topk": int(ref["logp"].shape[1]),
                          "mean_mass_in_topk": round(mass, 4), "out": a.out}))
        return 0
    ref = torch.load(a.ref)
    rows: List[Dict] = []
    allkl = []
    for f in a.logits:
        d = torch.load(f)
        if "ids_in" in ref and ref["ids_in"].numel() and d.get("ids") is not None:
            if list(ref["ids_in"].tolist())[:len(d["ids"])] != list(d["ids"])[:ref["ids_in"].numel()]:
                print(json.dumps({"error": f"{f} was computed over other token ids than the reference"}))
                return 2
        kl = score(ref, d["logits"], a.skip)
        top1 = float((d["logits"][a.skip:kl.shape[0] + a.skip].argmax(-1) == ref["ids"][a.skip:kl.shape[0] + a.skip, 0].long()).float().mean())
        rows.append({"file": f, "positions": int(kl.numel()), "kl_mean": round(float(kl.mean()), 6),
                     "kl_max": round(float(kl.max()), 6), "top1_agreement": round(top1, 4)})
        allkl.append(kl)
    cat = torch.cat(allkl)
    print(json.dumps({"kl_mean": round(float(cat.mean()), 6), "kl_max": round(float(cat.max()), 6), "sequences": rows}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
