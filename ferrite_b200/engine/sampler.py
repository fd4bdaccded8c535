"""Host-side token sampling: temperature, top-k, top-p, min-p, presence / frequency / repetition penalties, a seeded
SplitMix64 generator, and speculative acceptance against point-mass drafts.

Counterparts in the reference: `dist` / `draw_excluding` / `penalize` / `sample` (`crates/fe-model/src/sched.rs:2103-2200`)
and `Sampler::{sample_bf16, sample_bf16_banning, spec_accept}` + `Rng` (`crates/fe-server/src/sampler.rs:189`). Greedy
requests never come here: the device argmax kernel picks their tokens.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

_M64 = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.s = seed & _M64

    def next_u64(self) -> int:
        self.s = (self.s + 0x9E3779B97F4A7C15) & _M64
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        return z ^ (z >> 31)

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))


@dataclass
class Sampling:
    temperature: float = 0.0        # 0 = greedy
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    max_tokens: int = 256
    stop_ids: List[int] = field(default_factory=list)
    banned_first: List[int] = field(default_factory=list)     # ids that may not open the reply (first-token stop ban)

    @property
    def argmax(self) -> bool:
        """Temperature 0: the pick is the arg-max of the (possibly penalised) logits."""
        return self.temperature <= 0.0

    @property
    def penalised(self) -> bool:
        return self.presence_penalty != 0 or self.frequency_penalty != 0 or self.repetition_penalty != 1.0

    @property
    def greedy(self) -> bool:
        """The device arg-max kernel may pick this request's tokens: temperature 0 and every penalty neutral (the
        reference's `greedy()`, `crates/fe-model/src/sched.rs:162`). A temperature-0 request with penalties takes the
        host sampler's arg-max, so its output does not depend on what else is in the batch."""
        return self.temperature <= 0.0 and not self.penalised


def penalize(logits: torch.Tensor, counts: Dict[int, int], s: Sampling, seen: Optional[Sequence[int]] = None,
             rep_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Presence and frequency penalties over the tokens generated so far (counts: id -> occurrences); the repetition
    penalty over the union of the prompt's tokens (`seen`) and the generated ones, as in the reference (`penalize`,
    `crates/fe-model/src/sched.rs:2158`). `rep_mask` (bool [vocab]) is that union kept up to date by the caller: with it
    a 100K-token prompt costs one vectorised pass per token instead of a set union."""
    if not s.penalised:
        return logits
    out = logits.clone()
    if s.repetition_penalty != 1.0 and s.repetition_penalty > 0 and rep_mask is not None:
        out = torch.where(rep_mask, torch.where(out > 0, out / s.repetition_penalty, out * s.repetition_penalty), out)
    elif s.repetition_penalty != 1.0 and s.repetition_penalty > 0:
        rep = set(counts.keys())
        if seen:
            rep.update(int(t) for t in seen)
        rep = [t for t in rep if 0 <= t < out.numel()]
        if rep:
            ids = torch.tensor(sorted(rep), dtype=torch.long)
            v = out[ids]
            out[ids] = torch.where(v > 0, v / s.repetition_penalty, v * s.repetition_penalty)
    if counts and (s.presence_penalty != 0 or s.frequency_penalty != 0):
        ids = torch.tensor(list(counts.keys()), dtype=torch.long)
        cnt = torch.tensor(list(counts.values()), dtype=out.dtype)
        out[ids] = out[ids] - s.presence_penalty - s.frequency_penalty * cnt
    return out


def _native():
    """The C++ sampler (`csrc/host_sampler.cpp`) when the extension is built, else None."""
    from .._ext import host
    h = host()
    return h if h is not None and hasattr(h, "sample_probs") else None


def dist(logits: torch.Tensor, s: Sampling, banned: Sequence[int] = ()) -> torch.Tensor:
    """Probability vector after temperature, top-k, top-p and min-p (top-p is applied inside the top-k set). Runs in C++
    when the extension is built (no full sort of the vocabulary); the statements below are its definition."""
    h = _native()
    if h is not None and logits.device.type == "cpu":
        return h.sample_probs(logits.float().contiguous(), float(s.temperature), int(s.top_k or 0), float(s.top_p),
                              float(s.min_p), [int(b) for b in banned])
    lf = logits.float().clone()
    if len(banned):
        lf[torch.tensor(list(banned), dtype=torch.long)] = float("-inf")
    t = s.temperature if s.temperature > 0 else 1.0
    p = torch.softmax(lf / t, -1)
    if s.top_k and s.top_k < p.numel():
        kth = torch.topk(p, s.top_k).values[-1]
        p = torch.where(p >= kth, p, torch.zeros_like(p))
    if 0.0 < s.top_p < 1.0:
        sp, si = torch.sort(p, descending=True, stable=True)
        cum = torch.cumsum(sp, 0) / sp.sum()
        keep = (cum - sp / sp.sum()) < s.top_p            # keep tokens until the mass before them reaches top_p
        mask = torch.zeros_like(p, dtype=torch.bool)
        mask[si[keep]] = True
        p = torch.where(mask, p, torch.zeros_like(p))
    if s.min_p > 0.0:
        p = torch.where(p >= s.min_p * p.max(), p, torch.zeros_like(p))
    tot = p.sum()
    return p / tot if tot > 0 else torch.softmax(lf, -1)


def draw(p: torch.Tensor, rng: SplitMix64) -> int:
    """Inverse-CDF draw in index order (deterministic for a seed)."""
    h = _native()
    if h is not None and p.device.type == "cpu" and p.dtype == torch.float32:
        return int(h.sample_draw(p.contiguous(), rng.uniform(), -1))
    u = rng.uniform() * float(p.sum())
    c = torch.cumsum(p.double(), 0)
    i = int(torch.searchsorted(c, torch.tensor(u, dtype=torch.float64), right=True))
    return min(i, p.numel() - 1)


def draw_excluding(p: torch.Tensor, rng: SplitMix64, excluded: int) -> int:
    h = _native()
    if h is not None and p.device.type == "cpu" and p.dtype == torch.float32:
        # the generator advances only when there is something else to draw, as below
        if not (float(p.sum()) - float(p[excluded]) > 0):
            return excluded
        return int(h.sample_draw(p.contiguous(), rng.uniform(), int(excluded)))
    q = p.clone()
    q[excluded] = 0
    if float(q.sum()) <= 0:
        return excluded
    return draw(q / q.sum(), rng)


class Sampler:
    def __init__(self, s: Sampling, request_seed: int = 0, prompt: Optional[Sequence[int]] = None):
        self.s = s
        self.rng = SplitMix64(s.seed if s.seed is not None else request_seed)
        self.counts: Dict[int, int] = {}
        # prompt tokens count for the repetition penalty only
        self.seen = frozenset(int(t) for t in prompt) if (prompt is not None and s.repetition_penalty != 1.0) else None
        self.rep_mask: Optional[torch.Tensor] = None     # prompt and generated ids, built at the first penalised row

    def observe(self, tok: int) -> None:
        self.counts[tok] = self.counts.get(tok, 0) + 1
        if self.rep_mask is not None and 0 <= tok < self.rep_mask.numel():
            self.rep_mask[tok] = True

    def _penalized(self, logits: torch.Tensor) -> torch.Tensor:
        lf = logits.float().cpu()
        if self.s.repetition_penalty != 1.0 and self.s.repetition_penalty > 0:
            if self.rep_mask is None or self.rep_mask.numel() != lf.numel():
                ids = set(self.counts.keys()) | (set(self.seen) if self.seen else set())
                self.rep_mask = torch.zeros(lf.numel(), dtype=torch.bool)
                ids = [t for t in ids if 0 <= t < lf.numel()]
                if ids:
                    self.rep_mask[torch.tensor(ids, dtype=torch.long)] = True
        return penalize(lf, self.counts, self.s, self.seen, self.rep_mask)

    def probs(self, logits: torch.Tensor, first: bool = False) -> torch.Tensor:
        return dist(self._penalized(logits), self.s, self.s.banned_first if first else ())

    def sample(self, logits: torch.Tensor, first: bool = False) -> int:
        if self.s.argmax:
            lf = self._penalized(logits)
            if first and self.s.banned_first:
                lf = lf.clone()
                lf[torch.tensor(self.s.banned_first, dtype=torch.long)] = float("-inf")
            return int(lf.argmax())
        return draw(self.probs(logits, first), self.rng)

    def spec_accept(self, logits_rows: torch.Tensor, drafts: Sequence[int]) -> List[int]:
        """Walk a verified chain. logits_rows[i] is the target distribution after i accepted drafts. Greedy:
        accept while the draft equals the arg-max. Sampled: a draft (a point mass) is accepted with probability
        p(draft); on rejection the replacement is drawn from p with the draft excluded, which keeps the output
        distribution exactly the target's. Returns the tokens to emit (accepted drafts + one more)."""
        out: List[int] = []
        for i in range(len(drafts) + 1):
            row = logits_rows[i]
            if i == len(drafts):
                out.append(self.sample(row))
                break
            d = int(drafts[i])
            if self.s.argmax:
                t = self.sample(row)
                out.append(t)
                if t != d:
                    break
            else:
                p = self.probs(row)
                if self.rng.uniform() < float(p[d]):
                    out.append(d)
                else:
                    out.append(draw_excluding(p, self.rng, d))
                    break
            self.observe(out[-1])
        else:
            return out
        self.observe(out[-1])
        return out
