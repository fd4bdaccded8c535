"""`BatchEngine`: continuous batching over a slot-level step model, plus a deterministic fake model.

The model side is `StepModel`: a fixed number of cache slots, `forward(segments, logit_rows)` over any mix of
(slot, tokens) segments, `argmax` / `logits_host` for the requested rows, `reset_slot`. One scheduler thread owns the
model and every step (1) admits queued requests into free slots, reusing a slot whose cached history is a prefix of the
new prompt (only the rest is prefilled), (2) builds one forward: a decode row per generating request, then prompt chunks
within the model's row budget, (3) picks tokens (model argmax when every row is plain greedy, else host sampling) and
streams them, stopping on stop ids / `max_tokens` / cancellation.

This is the small engine behind `--engine ferrite-batch` / `--engine fake`: no speculation, no parking. Counterpart of
the reference's `crates/fe-server/src/batch.rs` (`StepModel` `:23`, `BatchConfig` `:43`, `BatchEngine::spawn` `:68`,
`fake::FakeModel`, `reference` `:411`, `generate` `:506`).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..engine.sampler import Sampler
from .engine_api import EngineBase, EngineInfo, GenEvent, GenRequest, TokenSink


class StepModel:
    """A batched, slot-based forward pass."""

    def n_slots(self) -> int: raise NotImplementedError
    def max_ctx(self) -> int: raise NotImplementedError
    def max_rows(self) -> int: raise NotImplementedError
    def vocab(self) -> int: raise NotImplementedError

    def reset_slot(self, slot: int) -> None:
        """Empty a slot (its next token is position 0)."""
        raise NotImplementedError

    def forward(self, segs: Sequence[Tuple[int, Sequence[int]]], logit_rows: Sequence[int]) -> None:
        """Append `segs` = (slot, tokens) to their slots; compute logits for the listed rows (indices into the
        concatenation of all segments' tokens), in that order."""
        raise NotImplementedError

    def argmax(self, n: int) -> List[int]:
        """Greedy token for each of the first n logit rows of the last forward."""
        raise NotImplementedError

    def logits_host(self, n: int) -> torch.Tensor:
        """The first n logit rows of the last forward, [n, vocab] fp32 on the host."""
        raise NotImplementedError


@dataclass
class BatchConfig:
    name: str = "ferrite"
    prefill_chunk: int = 0          # prompt rows per request per step (0 = the model's max_rows)


@dataclass
class _Slot:
    busy: bool = False
    hist: List[int] = field(default_factory=list)      # tokens in this slot's cache since the last reset
    last_used: int = 0


@dataclass
class _Job:
    req: GenRequest
    sink: TokenSink
    slot: int = -1
    pending: List[int] = field(default_factory=list)   # prompt tokens not yet forwarded
    next_token: Optional[int] = None
    out: List[int] = field(default_factory=list)
    cached: int = 0
    sampler: Optional[Sampler] = None
    t0: float = 0.0
    t_prompt: float = 0.0


class BatchEngine(EngineBase):
    def __init__(self, cfg: BatchConfig, factory: Callable[[], StepModel], model_name: str = "model"):
        """Starts the scheduler thread; `factory` builds the model ON that thread (a CUDA context created there stays
        current). Returns once the model is up, or raises the factory's error."""
        self.cfg, self.model_name = cfg, model_name
        self.q: "queue.Queue[Optional[_Job]]" = queue.Queue()
        self._info: Optional[EngineInfo] = None
        self._err: Optional[str] = None
        self._dead: Optional[str] = None
        self.stats = {"steps": 0, "prompt_tokens": 0, "cached_tokens": 0, "tokens": 0, "requests": 0}
        self._n_active = 0
        up = threading.Event()

        def run():
            try:
                model = factory()
                self._info = EngineInfo(cfg.name, model_name, model.n_slots(), model.max_ctx(), model.vocab())
            except Exception as e:                                   # noqa: BLE001
                self._err = repr(e)
                up.set()
                return
            up.set()
            try:
                self._loop(model)
            except Exception as e:                                   # noqa: BLE001
                self._dead = f"batch engine thread died: {e!r}"
        self._thread = threading.Thread(target=run, name="fe-batch", daemon=True)
        self._thread.start()
        up.wait()
        if self._err:
            raise RuntimeError(f"batch engine: {self._err}")

    # ---- Engine surface ---------------------------------------------------------------------------------------------
    def info(self) -> EngineInfo:
        return self._info

    def submit(self, req: GenRequest, sink: TokenSink) -> None:
        if self._dead or not self._thread.is_alive():
            sink(GenEvent("error", message="the batch engine has stopped"))
            return
        self.q.put(_Job(req, sink, t0=time.time()))

    def dead(self) -> Optional[str]:
        return self._dead

    def load(self) -> Dict[str, int]:
        return {"running": self._n_active, "queued": self.q.qsize()}

    def metrics(self) -> Dict[str, float]:
        return {k: float(v) for k, v in self.stats.items()}

    def shutdown(self) -> None:
        self.q.put(None)
        self._thread.join(timeout=10)

    # ---- scheduler thread -------------------------------------------------------------------------------------------
    def _loop(self, m: StepModel) -> None:
        slots = [_Slot() for _ in range(m.n_slots())]
        waiting: List[_Job] = []
        active: List[_Job] = []
        tick = 0
        chunk = self.cfg.prefill_chunk or m.max_rows()
        while True:
            # intake
            try:
                job = self.q.get(timeout=None if not (active or waiting) else 0)
                if job is None:
                    return
                waiting.append(job)
                while True:
                    job = self.q.get_nowait()
                    if job is None:
                        return
                    waiting.append(job)
            except queue.Empty:
                pass
            # admission: the free slot whose history is the longest proper prefix of the prompt, else the least
            # recently used free slot (reset)
            still = []
            for job in waiting:
                if job.req.cancel.is_set():
                    job.sink(GenEvent("finish", reason="cancelled"))
                    continue
                free = [i for i, s in enumerate(slots) if not s.busy]
                if not free:
                    still.append(job)
                    continue
                ids = job.req.ids
                if len(ids) + 1 > m.max_ctx():
                    job.sink(GenEvent("error", message=f"prompt of {len(ids)} tokens exceeds the context of {m.max_ctx()}"))
                    continue

                def prefix_len(i):
                    h = slots[i].hist
                    return len(h) if 0 < len(h) < len(ids) and ids[:len(h)] == h else -1
                best = max(free, key=lambda i: (prefix_len(i), -slots[i].last_used))
                keep = prefix_len(best)
                if keep <= 0:
                    m.reset_slot(best)
                    slots[best].hist = []
                    keep = 0
                tick += 1
                slots[best].busy, slots[best].last_used = True, tick
                job.slot, job.cached, job.pending = best, keep, list(ids[keep:])
                job.sampler = Sampler(job.req.sampling, request_seed=tick, prompt=ids)
                self.stats["cached_tokens"] += keep
                self.stats["requests"] += 1
                active.append(job)
            waiting = still
            self._n_active = len(active)
            if not active:
                continue
            # one forward: decode rows first, then prompt chunks inside the row budget
            segs: List[Tuple[int, List[int]]] = []
            rows: List[int] = []
            owners: List[Tuple[_Job, bool]] = []                     # (job, this row yields a token)
            r = 0
            budget = m.max_rows()
            for job in active:
                if job.req.cancel.is_set():
                    continue
                if not job.pending and job.next_token is not None and budget > 0:
                    segs.append((job.slot, [job.next_token]))
                    rows.append(r)
                    owners.append((job, True))
                    r += 1
                    budget -= 1
            for job in active:
                if job.pending and budget > 0 and not job.req.cancel.is_set():
                    n = min(len(job.pending), chunk, budget)
                    toks, job.pending = job.pending[:n], job.pending[n:]
                    segs.append((job.slot, toks))
                    last = not job.pending
                    if last:
                        rows.append(r + n - 1)
                    owners.append((job, last))
                    r += n
                    budget -= n
                    self.stats["prompt_tokens"] += n
            done: List[Tuple[_Job, str]] = [(j, "cancelled") for j in active if j.req.cancel.is_set()]
            if segs:
                m.forward(segs, rows)
                self.stats["steps"] += 1
                for slot, toks in segs:
                    slots[slot].hist.extend(toks)
                yielding = [j for j, y in owners if y]
                greedy = all(j.req.sampling.greedy and not (j.req.sampling.banned_first and not j.out) for j in yielding)
                picks = m.argmax(len(yielding)) if (greedy and yielding) else None
                logits = None if greedy or not yielding else m.logits_host(len(yielding))
                for k, job in enumerate(yielding):
                    if not job.out and not job.t_prompt:
                        job.t_prompt = time.time()
                    t = int(picks[k]) if picks is not None else job.sampler.sample(logits[k], first=not job.out)
                    job.sampler.observe(t)
                    s = job.req.sampling
                    if t in s.stop_ids:
                        done.append((job, "stop"))
                        continue
                    job.out.append(t)
                    self.stats["tokens"] += 1
                    job.sink(GenEvent("tokens", tokens=[t]))
                    job.next_token = t
                    if len(job.out) >= s.max_tokens or len(slots[job.slot].hist) + 1 >= m.max_ctx():
                        done.append((job, "length"))
                    elif job.req.guard is not None:
                        g = job.req.guard([t])
                        if isinstance(g, str) and g:
                            done.append((job, g))
            for job, reason in done:
                if job in active:
                    active.remove(job)
                    slots[job.slot].busy = False
                    now = time.time()
                    job.sink(GenEvent("finish", reason=reason, timings={
                        "prompt_n": len(job.req.ids) - job.cached, "cache_n": job.cached, "predicted_n": len(job.out),
                        "prompt_ms": 1e3 * ((job.t_prompt or now) - job.t0), "predicted_ms": 1e3 * (now - (job.t_prompt or now))}))
            self._n_active = len(active)


# ---- a deterministic CPU "model": next token = f(sum of the history, its length) -------------------------------------

def fake_next_token(total: int, length: int, text_vocab: int, eos: int, eos_period: int) -> int:
    if length > 40 and total % eos_period == 0:
        return eos
    return (total * 31 + length) % (text_vocab - 2) + 2


def fake_reference(prompt: Sequence[int], max_tokens: int, text_vocab: int, eos: int, eos_period: int):
    """What a solo greedy run of the fake produces: (tokens, finish reason)."""
    total, length, out = sum(int(t) for t in prompt), len(prompt), []
    while True:
        t = fake_next_token(total, length, text_vocab, eos, eos_period)
        if t == eos:
            return out, "stop"
        out.append(t)
        if len(out) >= max_tokens:
            return out, "length"
        total += t
        length += 1


class FakeModel(StepModel):
    """Slots that remember (sum, length) of their history; logits put all the mass on `fake_next_token`."""

    def __init__(self, n_slots: int = 4, max_ctx: int = 4096, max_rows: int = 512, vocab: int = 300, text_vocab: int = 256,
                 eos: int = 1, eos_period: int = 97):
        self._n, self._ctx, self._rows, self._vocab = n_slots, max_ctx, max_rows, vocab
        self.text_vocab, self.eos, self.eos_period = text_vocab, eos, eos_period
        self.state = [[0, 0] for _ in range(n_slots)]
        self.last: List[int] = []
        self.log: List[Tuple[int, int]] = []          # (rows, logit rows) of every forward, for the tests

    def n_slots(self): return self._n
    def max_ctx(self): return self._ctx
    def max_rows(self): return self._rows
    def vocab(self): return self._vocab

    def reset_slot(self, slot):
        self.state[slot] = [0, 0]

    def forward(self, segs, logit_rows):
        want, r, picks = set(logit_rows), 0, {}
        assert sum(len(t) for _, t in segs) <= self._rows
        for slot, toks in segs:
            for t in toks:
                st = self.state[slot]
                st[0] += int(t)
                st[1] += 1
                assert st[1] <= self._ctx
                if r in want:
                    picks[r] = fake_next_token(st[0], st[1], self.text_vocab, self.eos, self.eos_period)
                r += 1
        self.last = [picks[i] for i in logit_rows]
        self.log.append((r, len(logit_rows)))

    def argmax(self, n):
        return self.last[:n]

    def logits_host(self, n):
        out = torch.full((n, self._vocab), -30.0)
        for i, t in enumerate(self.last[:n]):
            out[i, t] = 30.0
        return out


class EngineStepModel(StepModel):
    """`engine.engine.Engine` behind the step-model surface (reference: `FeModel`, `crates/fe-server/src/ferrite.rs:20-30`)."""

    def __init__(self, engine):
        self.eng = engine
        self._logits = None
        self._picks = None

    def n_slots(self): return self.eng.ecfg.n_slots
    def max_ctx(self): return self.eng.ecfg.max_ctx
    def max_rows(self): return min(self.eng.ecfg.max_step_rows, self.eng.ecfg.prefill_chunk)
    def vocab(self): return self.eng.full_cfg.vocab

    def reset_slot(self, slot):
        self.eng.reset_slot(slot)

    def forward(self, segs, logit_rows):
        from ..engine.executor import Segment
        want = set(logit_rows)
        out, r = [], 0
        for slot, toks in segs:
            n = len(toks)
            last = (r + n - 1) in want
            assert not any(i in want for i in range(r, r + n - 1)), "only the last row of a segment yields logits"
            out.append(Segment(slot, self.eng.slot_len[slot], list(toks), "last" if last else "none"))
            r += n
        self._logits, self._picks, _ = self.eng.forward(out, commit=True, greedy=False)

    def argmax(self, n):
        return self._logits[:n].float().argmax(-1).tolist()

    def logits_host(self, n):
        return self._logits[:n].float().cpu()
