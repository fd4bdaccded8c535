"""Command line of the engine (no server): `python -m ferrite_b200.cli <command> ...`

    generate   --preset 27b [--model DIR] --prompt "text" | --ids 1,2,3  [--max-tokens 64]    greedy text and tok/s
    logits     --preset 27b [--model DIR] --ids-file ids.txt --out logits.pt [--chunk 256] [--schedule plain|stagger|split|mix]
    logits-test --preset tiny [--tokens 200] [--chunk 64]     the same logits whatever the step schedule
    sched-test --preset tiny [--requests 6]      every request through the scheduler together == the same request alone
    park-test  --preset tiny                     a parked conversation resumed from the prompt cache == recomputed from scratch

Common: `--device cuda|cpu`, `--layers N` (cut the model), `--weights bf16|nvfp4|...`, `--spec N` (draft depth for the
scheduler commands). `--model DIR` loads a checkpoint directory (safetensors bf16 / ModelOpt NVFP4 / EXL3 / GGUF) and its
tokenizer; without it the weights are seeded random and ids stand for text.

Counterpart of the reference's `ferrite generate | logits | sched-test | park-test` (`crates/fe-cli/src/main.rs:926-970`);
`logits` writes what `utils/kl.py` and external KL tools read.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional

import torch


def build_engine(a, n_slots: int = 1, max_ctx: int = 4096):
    from .config import PRESETS, EngineConfig, ModelConfig, scaled
    from .engine.engine import Engine
    import os
    weights = None
    if a.model:
        cfg_path = os.path.join(a.model, "config.json")
        cfg = ModelConfig.from_hf(cfg_path) if os.path.exists(cfg_path) else PRESETS[a.preset]()
        files = sorted(os.listdir(a.model))
        if any(f.endswith(".safetensors") for f in files):
            from .formats.loader import load_model_weights
            weights = load_model_weights(a.model, cfg)
        else:
            ggufs = [f for f in files if f.endswith(".gguf")]
            if not ggufs:
                raise SystemExit(f"{a.model}: no .safetensors and no .gguf file")
            from .formats import gguf as G
            from .formats.gguf_model import config_from_gguf, load_gguf_weights
            g = G.Gguf(os.path.join(a.model, ggufs[0]))
            cfg = config_from_gguf(g, cfg)
            g.close()
            weights = load_gguf_weights(os.path.join(a.model, ggufs[0]), cfg)
    else:
        cfg = PRESETS[a.preset]()
    from .server.tokenizer import load_tokenizer
    tok = load_tokenizer(a.model or None, cfg.vocab)              # byte tokenizer when the directory has none
    if a.layers:
        cfg = scaled(cfg, a.layers)
    ecfg = EngineConfig(n_slots=n_slots, max_ctx=max_ctx, weight_dtype=a.weights)
    eng = Engine(cfg, weights, ecfg, device=a.device or None, seed=a.seed)
    return cfg, eng, tok


def parse_ids(a, tok, vocab: int) -> List[int]:
    if a.ids:
        return [int(x) for x in a.ids.replace(" ", "").split(",") if x]
    return [t % vocab for t in tok.encode(a.prompt)]


def cmd_generate(a) -> int:
    cfg, eng, tok = build_engine(a, max_ctx=a.max_ctx)
    ids = parse_ids(a, tok, cfg.vocab)
    sync = (lambda: torch.cuda.synchronize()) if eng.device.type == "cuda" else (lambda: None)
    t0 = time.perf_counter()
    eng.prefill(0, ids[:-1]) if len(ids) > 1 else None
    sync()
    t1 = time.perf_counter()
    out: List[int] = []
    nxt, pos = ids[-1], len(ids) - 1
    from .engine.executor import Segment
    for _ in range(a.max_tokens):
        _, picks, _ = eng.forward([Segment(0, pos, [nxt], "last")], commit=True, greedy=True)
        nxt = int(picks[0][0])
        out.append(nxt)
        pos += 1
    sync()
    t2 = time.perf_counter()
    eng.check()
    print(json.dumps({"prompt_tokens": len(ids), "new_tokens": len(out), "ids": out,
                      "text": tok.decode(out),
                      "prefill_tok_s": round((len(ids) - 1) / max(1e-9, t1 - t0), 1),
                      "decode_tok_s": round(len(out) / max(1e-9, t2 - t1), 1)}))
    return 0


def scheduled_logits(eng, ids: List[int], chunk: int, schedule: str) -> torch.Tensor:
    """Per-position logits of `ids` on slot 0 under a step schedule that must not change them:
    plain    chunks of `chunk` rows
    stagger  chunks of varying sizes (chunk, 1, chunk / 2 + 1, 3, ...), so cuts land off the 32-row grid
    split    the same chunks, but a second request's chunk (other tokens, slot 1) rides in every step before them
    mix      every prompt chunk shares its step with a decode row of a request running on slot 1
    Reference: `ferrite logits` under `FE_LOG_SCHED=stagger|split|mix` (`crates/fe-cli/src/main.rs`)."""
    from .engine.executor import Segment
    sizes: List[int] = []
    left, k = len(ids), 0
    pattern = [chunk] if schedule in ("plain", "split", "mix") else [chunk, 1, chunk // 2 + 1, 3]
    while left > 0:
        n = max(1, min(left, pattern[k % len(pattern)]))
        sizes.append(n)
        left -= n
        k += 1
    other = [(t * 7 + 3) % eng.full_cfg.vocab for t in ids]
    if schedule == "mix":
        eng.reset_slot(1)
        eng.prefill(1, other[:5])
    rows, i = [], 0
    for step, n in enumerate(sizes):
        segs = [Segment(0, i, ids[i:i + n], "all")]
        if schedule == "split":
            segs = [Segment(1, i, other[i:i + n], "none")] + segs
        elif schedule == "mix":
            segs = [Segment(1, eng.slot_len[1], [other[(5 + step) % len(other)]], "last")] + segs
        lg, _, lrows = eng.forward(segs, greedy=False)
        first = next(j for j, r in enumerate(lrows) if r >= sum(len(s.tokens) for s in segs[:-1]))
        rows.append(lg[first:first + n].float().cpu().clone())
        i += n
    return torch.cat(rows)


def cmd_logits(a) -> int:
    cfg, eng, tok = build_engine(a, n_slots=2, max_ctx=a.max_ctx)
    with open(a.ids_file, "r", encoding="utf-8") as f:
        ids = [int(x) for x in f.readline().replace(" ", "").split(",") if x]
    logits = scheduled_logits(eng, ids, a.chunk, a.schedule)
    torch.save({"ids": ids, "logits": logits, "model": cfg.name, "weights": a.weights}, a.out)
    eng.check()
    print(json.dumps({"positions": len(ids), "vocab": int(logits.shape[1]), "out": a.out,
                      "finite": bool(torch.isfinite(logits).all())}))
    return 0


def cmd_logits_test(a) -> int:
    """The logits of a seeded prompt under every step schedule against the plain one: chunk cuts, a neighbour in the step
    and a decode row sharing the step must leave every row's logits where they were (to the kernels' batch invariance:
    bit for bit on the fp32 CPU engine, `--tol` elsewhere)."""
    cfg, eng, _ = build_engine(a, n_slots=2, max_ctx=a.max_ctx)
    g = torch.Generator().manual_seed(a.seed + 3)
    ids = torch.randint(1, cfg.vocab, (a.tokens,), generator=g).tolist()
    ref = scheduled_logits(eng, ids, a.chunk, "plain")
    out = {}
    for sched in ("stagger", "split", "mix"):
        eng.reset_slot(0)
        got = scheduled_logits(eng, ids, a.chunk, sched)
        out[sched] = float((got - ref).abs().max())
    eng.check()
    ok = all(v <= a.tol for v in out.values())
    print(json.dumps({"tokens": len(ids), "chunk": a.chunk, "max_abs_diff": out, "tol": a.tol, "ok": ok}))
    return 0 if ok else 1


def _prompts(cfg, n: int, seed: int, lo: int = 9, hi: int = 90) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi, (n,), generator=g).tolist()
    return [torch.randint(1, cfg.vocab, (ln,), generator=g).tolist() for ln in lens]


def cmd_sched_test(a) -> int:
    """Requests of different lengths, submitted together into fewer slots than requests, must each produce the tokens
    that the same request produces alone on a fresh slot (greedy): batching, chunked prompts, slot reuse, parking and
    speculation change the schedule, never the text. Reference `run_sched_test` (`crates/fe-cli/src/main.rs:1000`)."""
    from .engine.sampler import Sampling
    from .engine.scheduler import SchedOptions, Scheduler, generate
    cfg, eng, _ = build_engine(a, n_slots=a.slots, max_ctx=a.max_ctx)
    prompts = _prompts(cfg, a.requests, a.seed + 1)
    prompts[-1] = prompts[0] + prompts[-1][:7]                    # one request extends another: prefix sharing / resume
    samp = Sampling(max_tokens=a.max_tokens)
    alone = []
    for p in prompts:
        alone.append(eng.generate(p, a.max_tokens, slot=0))
    eng.reset_slot(0)
    sched = Scheduler(eng, SchedOptions(spec=a.spec, arrival_ms=0))
    t0 = time.perf_counter()
    together = generate(sched, prompts, samp)
    dt = time.perf_counter() - t0
    eng.check()
    bad = [i for i, (x, y) in enumerate(zip(alone, together)) if x != y]
    print(json.dumps({"requests": len(prompts), "slots": a.slots, "spec": a.spec, "mismatched": bad,
                      "steps": sched.stats.get("steps"), "cached_tokens": sched.stats.get("cached_tokens"),
                      "tok_s": round(sum(map(len, together)) / max(1e-9, dt), 1), "ok": not bad}))
    return 0 if not bad else 1


def cmd_park_test(a) -> int:
    """A conversation is run, pushed out of its only slot by another one (so it is parked: its recurrent-state snapshot
    and its KV pages leave the slot), then continued. The continuation must (1) resume from the parked snapshot instead of
    recomputing the prompt and (2) produce the tokens of a from-scratch run. Reference `run_park_test`
    (`crates/fe-cli/src/main.rs:1090`)."""
    from .engine.sampler import Sampling
    from .engine.scheduler import SchedOptions, Scheduler, generate
    cfg, eng, _ = build_engine(a, n_slots=1, max_ctx=a.max_ctx)
    g = torch.Generator().manual_seed(a.seed + 2)
    first = torch.randint(1, cfg.vocab, (70,), generator=g).tolist()
    other = torch.randint(1, cfg.vocab, (30,), generator=g).tolist()
    turn2 = first + torch.randint(1, cfg.vocab, (5,), generator=g).tolist()
    want = eng.generate(turn2, a.max_tokens, slot=0)
    eng.reset_slot(0)
    sched = Scheduler(eng, SchedOptions(spec=a.spec, arrival_ms=0))
    samp = Sampling(max_tokens=a.max_tokens)
    generate(sched, [first], Sampling(max_tokens=4), snapshots=[[64]])
    generate(sched, [other], Sampling(max_tokens=4))              # takes the slot: the first conversation is parked
    parked = len(sched.park)
    before = sched.stats["cached_tokens"]
    got = generate(sched, [turn2], samp)[0]
    resumed = sched.stats["cached_tokens"] - before
    eng.check()
    ok = parked >= 1 and resumed == 64 and got == want
    print(json.dumps({"parked_entries": parked, "resumed_tokens": resumed, "same_text": got == want, "ok": ok}))
    return 0 if ok else 1


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="ferrite_b200.cli", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p, max_tokens: int):
        p.add_argument("--preset", default="tiny", help="tiny | tiny-mla | 27b | moe80b | mla671b | drafter")
        p.add_argument("--model", default="", help="checkpoint directory (config.json + safetensors, or a .gguf)")
        p.add_argument("--layers", type=int, default=0)
        p.add_argument("--weights", default="bf16")
        p.add_argument("--device", default="")
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--max-ctx", type=int, default=4096)
        p.add_argument("--max-tokens", type=int, default=max_tokens)
        return p

    p = common(sub.add_parser("generate"), 64)
    p.add_argument("--prompt", default="Hello")
    p.add_argument("--ids", default="")
    p.set_defaults(fn=cmd_generate)
    p = common(sub.add_parser("logits"), 0)
    p.add_argument("--ids-file", required=True, help="one line of comma-separated token ids")
    p.add_argument("--out", required=True)
    p.add_argument("--chunk", type=int, default=256)
    p.add_argument("--schedule", default="plain", choices=["plain", "stagger", "split", "mix"])
    p.set_defaults(fn=cmd_logits)
    p = common(sub.add_parser("logits-test"), 0)
    p.add_argument("--tokens", type=int, default=200)
    p.add_argument("--chunk", type=int, default=64)
    p.add_argument("--tol", type=float, default=1e-4)
    p.set_defaults(fn=cmd_logits_test)
    p = common(sub.add_parser("sched-test"), 12)
    p.add_argument("--requests", type=int, default=6)
    p.add_argument("--slots", type=int, default=3)
    p.add_argument("--spec", type=int, default=0)
    p.set_defaults(fn=cmd_sched_test)
    p = common(sub.add_parser("park-test"), 6)
    p.add_argument("--spec", type=int, default=0)
    p.set_defaults(fn=cmd_park_test)
    a = ap.parse_args(argv)
    with torch.no_grad():
        return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
