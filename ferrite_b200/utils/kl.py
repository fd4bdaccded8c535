"""KL harness: divergence of a quantised engine's next-token distributions from the bf16 engine's on the same weights
and the same prompt (the role of the reference's `tools/kl.sh` + `kl_perseq.py`, which score an engine's `logits` dump
against a stored bf16 reference).

    python -m ferrite_b200.utils.kl --model 27b --layers 16 --dtype nvfp4 --tokens 512

Prints one JSON line: mean / max per-position KL(bf16 || quantised) in nats over `--tokens` positions of a seeded
uniform-random prompt, and the top-1 agreement. Both engines are built from the same seeded random-init weights.
`--ref dequantised` scores against a bf16 engine over the DEQUANTISED weights (kernel + activation error only, the
quantisation error of the weights themselves taken out); `--rows decode` scores one-row decode steps.
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
    ap.add_argument("--dtype", default="nvfp4", choices=["nvfp4", "nvfp4-w4a4", "nvfp4-a16", "fp8-block", "exl3", "bf16"])
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8", "int6", "int4", "fp8h", "int6h", "int4h"],
                    help="KV cache format of the tested engine")
    ap.add_argument("--device", default="cuda", help="cuda, or cpu for the fp32 statements (weight formats then decode to dense)")
    ap.add_argument("--ref", default="bf16", choices=["bf16", "dequantised"],
                    help="reference engine: bf16 on the original weights, or bf16 on the dequantised weights of the tested engine")
    ap.add_argument("--rows", default="prefill", choices=["prefill", "decode"], help="score prompt chunks or one-row decode steps")
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
    dev = a.device
    w = init_weights(cfg, seed=a.seed, dtype=torch.bfloat16, device=dev)
    prompt = torch.randint(0, cfg.vocab, (a.tokens,), generator=torch.Generator().manual_seed(99)).tolist()
    outs = {}

    def logits_of(eng):
        if a.rows == "decode":
            # one row per step: the few-row kernels (what a decode step runs) instead of the prompt GEMMs
            rows = []
            for i, t in enumerate(prompt):
                lg, _, _ = eng.forward([Segment(0, i, [t], "last")], greedy=False)
                rows.append(lg.float().cpu())
            return torch.cat(rows)
        # two chunks, so the second one reads the first through the (possibly quantised) cache
        half = a.tokens // 2
        l1, _, _ = eng.forward([Segment(0, 0, prompt[:half], "all")], greedy=False)
        l1 = l1.float().cpu()
        l2, _, _ = eng.forward([Segment(0, half, prompt[half:], "all")], greedy=False)
        return torch.cat([l1, l2.float().cpu()])

    eng = Engine(cfg, dict(w), EngineConfig(n_slots=1, max_ctx=a.tokens + 64, weight_dtype=a.dtype, kv_dtype=a.kv), device=dev)
    outs["test"] = logits_of(eng)
    if a.ref == "dequantised":
        # the reference multiplies the very values the codes stand for (the dequantised copies the quantised engine keeps),
        # in bf16 on the 16-bit kernels: what is left is the error of the quantised kernels and of their activation handling
        from ..ops.qweight import QWeight

        def dense_of(v):
            if isinstance(v, torch.Tensor):
                return v
            if isinstance(v, QWeight) and v.dense is not None:
                return v.dense
            return v.dequantize(torch.bfloat16).to(dev)          # EXL3 / GGUF / stacked parts: host decode of the codes
        w = {k: dense_of(v) for k, v in eng.ex.w.items() if isinstance(v, torch.Tensor) or hasattr(v, "dequantize") or isinstance(v, QWeight)}
    del eng
    torch.cuda.empty_cache()
    eng = Engine(cfg, dict(w), EngineConfig(n_slots=1, max_ctx=a.tokens + 64), device=dev)
    outs["ref"] = logits_of(eng)
    del eng
    torch.cuda.empty_cache()
    kl = kl_rows(outs["ref"], outs["test"])
    agree = (outs["ref"].argmax(-1) == outs["test"].argmax(-1)).float().mean().item()
    print(json.dumps({"model": cfg.name, "layers": cfg.n_layers, "dtype": a.dtype, "kv": a.kv, "reference": a.ref, "rows": a.rows, "positions": a.tokens,
                      "kl_mean": kl.mean().item(), "kl_max": kl.max().item(), "top1_agreement": agree,
                      "data": "seeded uniform-random prompt, random-init weights N(0, 0.02)"}))


if __name__ == "__main__":
    main()
