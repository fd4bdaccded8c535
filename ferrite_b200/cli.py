"""Command line of the engine (no server): `python -m ferrite_b200.cli <command> ...`

    generate   --preset 27b [--model DIR] --prompt "text" | --ids 1,2,3  [--max-tokens 64]    greedy text and tok/s
    logits     --preset 27b [--model DIR] --ids-file ids.txt --out logits.pt [--chunk 256] [--schedule plain|stagger|split|mix]
    logits-test --preset tiny [--tokens 200] [--chunk 64]     the same logits whatever the step schedule
    sched-test --preset tiny [--requests 6]      every request through the scheduler together == the same request alone
    park-test  --preset tiny                     a parked conversation resumed from the prompt cache == recomputed from scratch
    tree-test  --preset tiny [--nodes 7]         greedy text through verify trees (true chain + decoy branches) == plain decode
    df-snaptest --preset tiny [--tokens 300] [--window 0]   block drafter: drafts after save / absorb more / restore == before
    selftest   [--preset tiny]                   device facts, engine logits against the fp32 oracle model, bit-stable repeats
    bench      --preset 27b [--lens 2048,8192] [--dec 64] [--slots 4]   prefill and decode tok/s per length, then N streams
    gemm-bench [microbench arguments]            the GEMM / GEMV microbenchmarks (`utils/microbench.py`)

Launched under `python -m torch.distributed.run --nproc-per-node N` every rank runs the same command in lockstep over a
tensor-parallel engine (greedy picks are the same on every rank); rank 0 prints.

Common: `--device cuda|cpu`, `--layers N` (cut the model), `--weights bf16|nvfp4|...`, `--spec N` (draft depth for the
scheduler commands). `--model DIR` loads a checkpoint directory (safetensors bf16 / ModelOpt NVFP4 / EXL3 / GGUF) and its
tokenizer; without it the weights are seeded random and ids stand for text.

Counterpart of the reference's `ferrite selftest | gemm-bench | generate | logits | bench | sched-test | park-test |
tree-test | df-snaptest` (`crates/fe-cli/src/main.rs:926-970`; its `follow` is what ranks above 0 of the server do);
`logits` writes what `utils/kl.py` and external KL tools read.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional

import torch


def tp_from_env(a):
    """The tensor-parallel group of a lockstep launch (WORLD_SIZE > 1 in the environment), else None."""
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return None
    import torch.distributed as dist

    from .parallel.tp import TensorParallel
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available() and a.device != "cpu"
    if on_gpu:
        torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not dist.is_initialized():
        dist.init_process_group("nccl" if on_gpu else "gloo", **({"device_id": torch.device("cuda", local)} if on_gpu else {}))
    a.device = f"cuda:{local}" if on_gpu else "cpu"
    return TensorParallel(dist.group.WORLD, a.device)


def say(obj) -> None:
    """One JSON line, from rank 0 only."""
    import os
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(obj), flush=True)


def build_engine(a, n_slots: int = 1, max_ctx: int = 4096, tap_layers=None):
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
    if tap_layers == "thirds" and not cfg.tap_layers:
        cfg.tap_layers = sorted({max(0, cfg.n_layers * (i + 1) // 4 - 1) for i in range(3)})
    tp = tp_from_env(a)
    ecfg = EngineConfig(n_slots=n_slots, max_ctx=max_ctx, weight_dtype=a.weights)
    eng = Engine(cfg, weights, ecfg, device=a.device or None, seed=a.seed, tp=tp)
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
    say({"prompt_tokens": len(ids), "new_tokens": len(out), "ids": out,
                      "text": tok.decode(out),
                      "prefill_tok_s": round((len(ids) - 1) / max(1e-9, t1 - t0), 1),
                      "decode_tok_s": round(len(out) / max(1e-9, t2 - t1), 1)})
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
    import os
    if int(os.environ.get("RANK", "0")) == 0:
        torch.save({"ids": ids, "logits": logits, "model": cfg.name, "weights": a.weights}, a.out)
    eng.check()
    say({"positions": len(ids), "vocab": int(logits.shape[1]), "out": a.out,
                      "finite": bool(torch.isfinite(logits).all())})
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
    say({"tokens": len(ids), "chunk": a.chunk, "max_abs_diff": out, "tol": a.tol, "ok": ok})
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
    say({"requests": len(prompts), "slots": a.slots, "spec": a.spec, "mismatched": bad,
                      "steps": sched.stats.get("steps"), "cached_tokens": sched.stats.get("cached_tokens"),
                      "tok_s": round(sum(map(len, together)) / max(1e-9, dt), 1), "ok": not bad})
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
    say({"parked_entries": parked, "resumed_tokens": resumed, "same_text": got == want, "ok": ok})
    return 0 if ok else 1


def _sync(eng):
    if eng.device.type == "cuda":
        torch.cuda.synchronize(eng.device)


def _plain_greedy(eng, slot: int, ids: List[int], n: int) -> List[int]:
    from .engine.executor import Segment
    eng.reset_slot(slot)
    if len(ids) > 1:
        eng.prefill(slot, ids[:-1])
    out, nxt, pos = [], ids[-1], len(ids) - 1
    for _ in range(n):
        _, picks, _ = eng.forward([Segment(slot, pos, [nxt], "last")], commit=True, greedy=True)
        nxt = int(picks[0][0])
        out.append(nxt)
        pos += 1
    return out


def decoy_tree(truth: List[int], nodes: int, vocab: int, rng: torch.Generator):
    """A verify tree of at most `nodes` draft rows around a known continuation: the true chain, cut short at a random
    depth, with wrong siblings hung beside its nodes (sometimes in front of the true child, so that the walk has to pick
    the second sibling). Returns (tokens, parents) of the draft rows in segment numbering (row 0 is the root)."""
    toks: List[int] = []
    pars: List[int] = []
    depth = int(torch.randint(0, max(1, min(len(truth), nodes)) + 1, (1,), generator=rng))
    parent = 0
    for d in range(depth):
        if len(toks) >= nodes:
            break
        wrong = (truth[d] + 1 + int(torch.randint(0, vocab - 1, (1,), generator=rng))) % vocab
        first_wrong = bool(torch.rand(1, generator=rng) < 0.4) and len(toks) + 2 <= nodes
        if first_wrong:
            toks.append(wrong)
            pars.append(parent)
        toks.append(truth[d])
        pars.append(parent)
        nxt = len(toks)                                  # row index of the true child (rows are 1-based after the root)
        if not first_wrong and len(toks) < nodes and bool(torch.rand(1, generator=rng) < 0.4):
            toks.append(wrong)
            pars.append(parent)
        parent = nxt
    return toks, pars


def cmd_tree_test(a) -> int:
    """Greedy decoding through verify trees against plain decoding: every round feeds the last token plus a tree of draft
    rows (`decoy_tree` over the known continuation), walks the target's picks from the root, commits the accepted path
    (`commit_tree`: recurrent state replayed along the path, KV rows moved into place). The text must be the plain one.
    Reference `cmd_tree_test` (`crates/fe-cli/src/main.rs:212`)."""
    from .engine.executor import Segment
    from .engine.scheduler import tree_walk
    cfg, eng, tok = build_engine(a, n_slots=2, max_ctx=a.max_ctx)
    ids = parse_ids(a, tok, cfg.vocab)
    truth = _plain_greedy(eng, 1, ids, a.max_tokens)
    eng.reset_slot(0)
    if len(ids) > 1:
        eng.prefill(0, ids[:-1])
    rng = torch.Generator().manual_seed(a.seed + 9)
    out: List[int] = []
    nxt, pos = ids[-1], len(ids) - 1
    rounds = drafted = tree_rounds = 0
    t_ver = t_com = 0.0
    while len(out) < a.max_tokens:
        d, par = decoy_tree(truth[len(out):], min(a.nodes, a.max_tokens - len(out) - 1), cfg.vocab, rng)
        toks, pars = [nxt] + d, [-1] + par
        chain = pars[1:] == list(range(len(d)))
        _sync(eng)
        t0 = time.perf_counter()
        _, picks, _ = eng.forward([Segment(0, pos, toks, "all", parents=None if chain else pars)], commit=False, greedy=True)
        got = [int(t) for t in picks[0].tolist()]
        _sync(eng)
        t1 = time.perf_counter()
        path, new = tree_walk(toks, pars, got)
        if chain:
            eng.commit_verified([len(new)])
        else:
            eng.commit_tree([path])
        _sync(eng)
        t_com += time.perf_counter() - t1
        t_ver += t1 - t0
        out += new
        pos += len(new)
        nxt = new[-1]
        rounds += 1
        tree_rounds += 0 if chain else 1
        drafted += len(d)
    out = out[:a.max_tokens]
    eng.check()
    same = out == truth
    say({"new_tokens": len(out), "rounds": rounds, "tokens_per_round": round(len(out) / max(1, rounds), 2),
         "tree_rounds": tree_rounds, "draft_rows": drafted, "verify_ms_per_round": round(1e3 * t_ver / max(1, rounds), 3),
         "commit_ms_per_round": round(1e3 * t_com / max(1, rounds), 3), "same_text": same, "ok": same})
    return 0 if same else 1


def cmd_df_snaptest(a) -> int:
    """The block drafter's window snapshot: absorb a prompt, draft, save the window, absorb more, restore, draft again. The
    second draft must equal the first. With `--window` below the token count the slot is rebuilt in between (its own
    context is bounded), the snapshot no longer fits and the restore must leave an empty drafter that drafts again after
    the next absorb, never stale rows. Reference `fe_dflash::snaptest` (`crates/fe-dflash/src/lib.rs`)."""
    from .engine.executor import Segment
    from .models.drafter import BlockDrafter, drafter_config_for
    cfg, eng, _ = build_engine(a, n_slots=1, max_ctx=a.max_ctx, tap_layers="thirds")
    full = eng.full_cfg
    drafter = BlockDrafter(drafter_config_for(full), target_hidden=full.hidden, n_taps=len(full.tap_layers), n_slots=1,
                           max_ctx=a.max_ctx, device=str(eng.device), block=8, window=a.window, ring=2 * a.window, tp=eng.tp)
    g = torch.Generator().manual_seed(a.seed + 4)
    ids = torch.randint(1, full.vocab, (a.tokens,), generator=g).tolist()
    half = max(2, a.tokens // 3)

    def feed(lo: int, hi: int) -> None:
        i = lo
        while i < hi:
            n = min(64, hi - i)
            eng.forward([Segment(0, i, ids[i:i + n], "none")], commit=True)
            drafter.absorb(0, ids[i:i + n], i, eng.taps)
            i += n
    feed(0, half)
    before = drafter.draft(0, ids[half], half, eng.taps, 8)
    base0 = drafter.base[0]
    blob = drafter.save_window(0)
    feed(half, a.tokens)
    rebuilt = drafter.base[0] != base0
    drafter.restore_window(0, blob)
    after = drafter.draft(0, ids[half], half, eng.taps, 8) if not rebuilt else []
    if rebuilt:
        # the snapshot's rows are gone: the drafter must have started over and must work again once it is fed
        empty = drafter.eng.slot_len[0] == 0 and drafter.last_feat[0] is None
        eng.reset_slot(0)
        feed(0, half)
        again = drafter.draft(0, ids[half], half, eng.taps, 8)
        ok = empty and again == before
    else:
        ok = after == before and len(before) > 0
    eng.check()
    say({"tokens": a.tokens, "window": a.window, "rebuilt_in_between": rebuilt, "draft": before, "same_after_restore": ok, "ok": ok})
    return 0 if ok else 1


def cmd_selftest(a) -> int:
    """Device facts, then the engine against the fp32 oracle model on a seeded prompt (chunked prompt rows and decode rows),
    then bit-stability: the same step twice gives the same bits, and the token of a decode row equals the token of the
    same row fed as the last row of a prompt chunk. Reference `ferrite selftest` (`crates/fe-model/src/selftest.rs`)."""
    from .engine.executor import Segment
    from .models.ref import RefModel
    from .models.weights import init_weights
    facts = {"device": "cpu"}
    if torch.cuda.is_available() and a.device != "cpu":
        pr = torch.cuda.get_device_properties(0)
        facts = {"device": pr.name, "capability": f"sm_{pr.major}{pr.minor}", "sms": pr.multi_processor_count,
                 "memory_gb": round(pr.total_memory / (1 << 30), 1),
                 "smem_optin": getattr(pr, "shared_memory_per_block_optin", None)}
    cfg, eng, _ = build_engine(a, n_slots=2, max_ctx=256)
    full = eng.full_cfg
    g = torch.Generator().manual_seed(a.seed + 5)
    ids = torch.randint(1, full.vocab, (48,), generator=g).tolist()
    checks = {}
    if a.model == "" and full.n_layers <= 12 and full.hidden <= 512:
        ref = RefModel(full, init_weights(full, seed=a.seed))
        want = ref.forward(ids, ref.new_state())
        want = want[0] if isinstance(want, tuple) else want
        got = torch.cat([scheduled_logits(eng, ids[:40], 32, "plain")] +
                        [eng.forward([Segment(0, 40 + i, [ids[40 + i]], "last")], greedy=False)[0][:1].float().cpu().clone()
                         for i in range(8)])
        err = float((got - want).abs().max())
        tol = 1e-3 if eng.dtype == torch.float32 else 0.06 * float(want.abs().max()) + 0.02
        checks["oracle_max_abs_err"] = err
        checks["oracle_ok"] = err <= tol and float(
            (got.argmax(-1) == want.argmax(-1)).float().mean()) >= (1.0 if eng.dtype == torch.float32 else 0.9)
    # the same decode step twice: the same bits
    eng.reset_slot(1)
    eng.prefill(1, ids[:20])
    rows = []
    for _ in range(2):
        lg, _, _ = eng.forward([Segment(1, 20, [ids[20]], "last")], commit=False, greedy=False)
        rows.append(lg[0].float().cpu().clone())
    checks["repeat_bit_equal"] = bool(torch.equal(rows[0], rows[1]))
    # a decode row against the same row as the last of a chunk: the same token
    eng.reset_slot(1)
    lg, _, _ = eng.forward([Segment(1, 0, ids[:21], "last")], commit=False, greedy=False)
    checks["chunk_row_same_token"] = int(lg[0].argmax()) == int(rows[0].argmax())
    if eng.tp is not None:
        eng.tp.selftest()
        checks["peer_exchange_ok"] = True
    eng.check()
    ok = all(v for k, v in checks.items() if k.endswith(("_ok", "_equal", "_token")))
    say({**facts, "model": full.name, "checks": checks, "ok": ok})
    if ok:
        say("selftest: all OK")
    return 0 if ok else 1


def cmd_bench(a) -> int:
    """Prefill and decode rates per prompt length on one slot, then the aggregate of `--slots` streams decoding together
    (512 tokens of context each). Wall-clock around synchronised steps: the number a user of the CLI sees. Reference
    `cmd_bench` (`crates/fe-cli/src/main.rs:627`)."""
    from .engine.executor import Segment
    lens = [int(x) for x in a.lens.split(",") if x]
    cfg, eng, _ = build_engine(a, n_slots=max(1, a.slots), max_ctx=max(max(lens), 512) + a.dec + 8)
    seed, ids = 7, []
    for _ in range(max(max(lens), 512)):
        seed = (seed * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        ids.append((1000 + (seed >> 33) % 30000) % cfg.vocab)
    rep = {"model": eng.full_cfg.name, "weights": a.weights, "lens": []}
    for ln in lens:
        eng.reset_slot(0)
        _sync(eng)
        t0 = time.perf_counter()
        _, picks, _ = eng.prefill(0, ids[:ln])
        nxt = int(picks[0][-1])
        _sync(eng)
        pf = time.perf_counter() - t0
        pos = ln
        for timed in (False, True):                       # one warm-up step (graph capture), then the timed ones
            _sync(eng)
            t0 = time.perf_counter()
            for _ in range(a.dec if timed else 1):
                _, picks, _ = eng.forward([Segment(0, pos, [nxt], "last")], commit=True, greedy=True)
                nxt = int(picks[0][0])
                pos += 1
            _sync(eng)
            dt = time.perf_counter() - t0
        rep["lens"].append({"len": ln, "prefill_tok_s": round(ln / pf, 1), "decode_tok_s": round(a.dec / dt, 2),
                            "ms_per_token": round(1e3 * dt / a.dec, 3)})
    if a.slots > 1:
        nxts, poss = [], []
        for s in range(a.slots):
            eng.reset_slot(s)
            _, picks, _ = eng.prefill(s, ids[:512])
            nxts.append(int(picks[0][-1]))
            poss.append(512)
        for timed in (False, True):
            _sync(eng)
            t0 = time.perf_counter()
            for _ in range(a.dec if timed else 1):
                segs = [Segment(s, poss[s], [nxts[s]], "last") for s in range(a.slots)]
                _, picks, _ = eng.forward(segs, commit=True, greedy=True)
                nxts = [int(t) for t in picks[0].tolist()]
                poss = [p + 1 for p in poss]
            _sync(eng)
            dt = time.perf_counter() - t0
        rep["streams"] = {"slots": a.slots, "tok_s_total": round(a.slots * a.dec / dt, 2),
                          "tok_s_per_stream": round(a.dec / dt, 2), "ms_per_step": round(1e3 * dt / a.dec, 3)}
    eng.check()
    say(rep)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["gemm-bench"]:
        from .utils import microbench
        sys.argv = ["microbench"] + (argv[1:] or ["gemm", "--m", "2048", "--n", "34816", "--k", "5120"])
        return microbench.main() or 0
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
    p = common(sub.add_parser("tree-test"), 48)
    p.add_argument("--prompt", default="Hello")
    p.add_argument("--ids", default="")
    p.add_argument("--nodes", type=int, default=7)
    p.set_defaults(fn=cmd_tree_test)
    p = common(sub.add_parser("df-snaptest"), 0)
    p.add_argument("--tokens", type=int, default=300)
    p.add_argument("--window", type=int, default=0)
    p.set_defaults(fn=cmd_df_snaptest)
    p = common(sub.add_parser("selftest"), 0)
    p.set_defaults(fn=cmd_selftest)
    p = common(sub.add_parser("bench"), 0)
    p.add_argument("--lens", default="2048,8192,32768")
    p.add_argument("--dec", type=int, default=64)
    p.add_argument("--slots", type=int, default=4)
    p.set_defaults(fn=cmd_bench)
    a = ap.parse_args(argv)
    with torch.no_grad():
        rc = a.fn(a)
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return rc


if __name__ == "__main__":
    sys.exit(main())
