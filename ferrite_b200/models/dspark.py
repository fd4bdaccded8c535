"""Markov (bigram-bias) drafting head with a confidence head, on top of a block drafter's per-step logits.

A block drafter scores `steps` future positions of a stream in one pass, each position blind to the tokens drafted
before it. The Markov head repairs that cheaply: the token picked at step i adds a low-rank bigram bias
`head @ emb[token]` to the logits of step i + 1 before its arg-max, so the draft is picked left to right while the
expensive pass stays parallel. Bias rows of the most frequent tokens are precomputed (`cache`); the others are computed
on the fly by one GEMV-like kernel per step. The confidence head then scores every drafted token from the drafter's
collapsed hidden row and the embedding of the token it followed; the scheduler cuts the draft where confidence drops.

Reference: `kernels/k-dspark/src/lib.rs:57-240` (kernels) and the `markov` module of `crates/fe-dspark` (host loop).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


class MarkovHead:
    def __init__(self, ops, head: torch.Tensor, emb: torch.Tensor, cached_tokens: Sequence[int] = (),
                 conf_w: Optional[torch.Tensor] = None, vocab_offset: int = 0):
        """head [V_local, rank] and emb [vocab, rank] in bf16; `cached_tokens`: token ids whose bias rows are kept
        resident; `conf_w` fp32 [d + rank]; `vocab_offset`: first global id of this rank's columns (tensor parallel)."""
        self.ops, self.head, self.emb, self.conf_w, self.col0 = ops, head, emb, conf_w, int(vocab_offset)
        dev = head.device
        self.slot_of = torch.full((emb.shape[0],), -1, dtype=torch.int32, device=dev)
        ids = torch.tensor(list(cached_tokens), dtype=torch.long, device=dev)
        if ids.numel():
            self.slot_of[ids] = torch.arange(ids.numel(), dtype=torch.int32, device=dev)
            all_slots = torch.full((ids.numel(),), -1, dtype=torch.int32, device=dev)
            self.cache = ops.markov_bias(head, emb, ids.to(torch.int32), all_slots)
        else:
            self.cache = torch.zeros(1, head.shape[0], dtype=torch.bfloat16, device=dev)

    def draft(self, anchors: torch.Tensor, step_logits: torch.Tensor) -> torch.Tensor:
        """anchors [rows] (the last accepted token of every stream), step_logits [steps, rows, V_local] fp32 ->
        draft [rows, steps + 1] int32 with draft[:, 0] = anchors."""
        ops = self.ops
        steps, rows = step_logits.shape[0], step_logits.shape[1]
        draft = torch.zeros(rows, steps + 1, dtype=torch.int32, device=anchors.device)
        draft[:, 0] = anchors.to(torch.int32)
        tok = draft[:, 0].contiguous()
        slot = self.slot_of[tok.long()]
        for i in range(steps):
            stage = ops.markov_bias(self.head, self.emb, tok, slot)
            tok, slot = ops.markov_step(draft, i, step_logits[i], stage, self.cache, slot, self.slot_of, col0=self.col0)
        return draft

    def confidence(self, xc: torch.Tensor, draft: torch.Tensor, block: int) -> torch.Tensor:
        """xc [streams * block, d]: the drafter's collapsed hidden rows; returns conf [streams, steps] fp32 logits."""
        steps = draft.shape[1] - 1
        return self.ops.conf_head(xc, self.emb, draft, self.conf_w, steps, block).view(draft.shape[0], steps)

    @staticmethod
    def cut(draft: torch.Tensor, conf: torch.Tensor, threshold: float) -> List[List[int]]:
        """Per stream: the drafted tokens up to (not including) the first whose confidence logit is below `threshold`."""
        out = []
        ok = (conf >= threshold).cpu()
        toks = draft[:, 1:].cpu()
        for s in range(draft.shape[0]):
            n = 0
            while n < ok.shape[1] and bool(ok[s, n]):
                n += 1
            out.append([int(t) for t in toks[s, :n]])
        return out
