"""KL harness: divergence of a quantised engine's next-token distributions from the bf16 engine's on the same weights
and the same prompt (the role of the reference's `tools/kl.sh` + `kl_perseq.py`, which score an engine's `logits` dump
against a stored bf16 reference).

    python -m ferrite_b200.utils.kl --model 27b --layers 16 --dtype nvfp4 --tokens 512

Prints one JSON line: mean / max per-position KL(bf16 || quantised) in nats over `--tokens` positions of a seeded
uniform-random prompt, and the top-1 agreement. Both engines are built from the same seeded random-init weights.
"""
from __future__ import annotations

import argparse
import json

import torch


def kl_rows(ref_logits: torch.Tensor, test_logits: torch.Tensor) -> torch.Tensor:
    lp = torch.log_softmax(ref_logits.float(), -1)
    lq = torch.log_softmax(test_logits.float(), -1)
    return (lp.exp() * (lp - lq)).sum(-1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="27b")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (0 = all)")
    ap.add_argument("--dtype", default="nvfp4", choices=["nvfp4", "nvfp4-a16", "fp8-block", "bf16"])
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8", "int4"], help="KV cache format of the tested engine")
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    from ..config import PRESETS, EngineConfig, scaled
    from ..engine.engine import Engine
    from ..engine.executor import Segment
    from ..models.weights import init_weights
    cfg = PRESETS[a.model]()
    if a.layers:
        cfg = scaled(cfg, a.layers)
    dev = "cuda"
    w = init_weights(cfg, seed=a.seed, dtype=torch.bfloat16, device=dev)
    prompt = torch.randint(0, cfg.vocab, (a.tokens,), generator=torch.Generator().manual_seed(99)).tolist()
    outs = {}
    for name, dt, kv in (("ref", "bf16", "bf16"), ("test", a.dtype, a.kv)):
        eng = Engine(cfg, dict(w), EngineConfig(n_slots=1, max_ctx=a.tokens + 64, weight_dtype=dt, kv_dtype=kv), device=dev)
        # two chunks, so the second one reads the first through the (possibly quantised) cache
        half = a.tokens // 2
        l1, _, _ = eng.forward([Segment(0, 0, prompt[:half], "all")], greedy=False)
        l1 = l1.float().cpu()
        l2, _, _ = eng.forward([Segment(0, half, prompt[half:], "all")], greedy=False)
        outs[name] = torch.cat([l1, l2.float().cpu()])
        del eng
        torch.cuda.empty_cache()
    kl = kl_rows(outs["ref"], outs["test"])
    agree = (outs["ref"].argmax(-1) == outs["test"].argmax(-1)).float().mean().item()
    print(json.dumps({"model": cfg.name, "layers": cfg.n_layers, "dtype": a.dtype, "kv": a.kv, "positions": a.tokens,
                      "kl_mean": kl.mean().item(), "kl_max": kl.max().item(), "top1_agreement": agree,
                      "data": "seeded uniform-random prompt, random-init weights N(0, 0.02)"}))


if __name__ == "__main__":
    main()
