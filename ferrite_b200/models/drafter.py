"""Block drafter for speculative decoding: a small attention-only decoder conditioned on hidden states tapped
from the target model, drafting a block of tokens in one forward pass.

Shape of the reference's DFlash2 drafter (`crates/fe-dflash/src/lib.rs`: 5 Qwen3-style layers, hidden 5120, 32Q/8KV
heads of 128, FFN 17408, reads feature taps of the target, block 16, draft window ring). Here it is an `Engine`
over an attention-only `ModelConfig`, plus one fusion matrix that maps the concatenated taps of the last committed
row into the drafter's input space. A block is drafted by feeding [last token, MASK x (n-1)] at the next n positions
(causal inside the block) with the fused features added to every row; row j predicts draft token j+1. Kept rows are
absorbed into the drafter's own KV cache with the features of the rows they came from.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..config import EngineConfig, ModelConfig
from ..engine.engine import Engine
from ..engine.executor import Segment
from ..engine.scheduler import Drafter, grow_tree


def drafter_config_for(target: ModelConfig) -> ModelConfig:
    """The block drafter's shape for a target: the reference's 5-layer drafter (`config.drafter_block`) for
    production-width targets, a two-layer miniature for the test presets; always the target's vocabulary."""
    from ..config import drafter_block
    if target.hidden >= 2048:
        cfg = drafter_block()
        cfg.vocab = target.vocab
        return cfg
    return ModelConfig(name="mini-drafter", hidden=128, inter=256, n_layers=2, full_attn_every=1, head_dim=32, n_q=4, n_kv=2,
                       rotary_dim=32, attn_gate=False, vocab=target.vocab, tie_embeddings=True)


class BlockDrafter(Drafter):
    def __init__(self, cfg: ModelConfig, target_hidden: int, n_taps: int, n_slots: int, max_ctx: int,
                 device: Optional[str] = None, seed: int = 1, block: int = 16, weights=None, mask_token: int = 0,
                 window: int = 0, ring: int = 0, weight_dtype: str = "bf16", tp=None):
        """`window` > 0 bounds the drafter's own context: its cache holds at most `ring` (default 2 x window) tokens in
        drafter-local positions; when a commit would run past the ring, the slot is rebuilt from the last `window`
        committed tokens and their features (one re-absorb of `window` rows per `ring - window` committed tokens) and
        goes on from there. The drafter then costs the same at 100K tokens of context as at 2K (reference: draft ring 4096 /
        window 2048, `crates/fe-dflash/src/lib.rs`). `weight_dtype`: the drafter's own weight format (the reference
        serves its drafter in 4 bits). `tp`: the target's tensor-parallel group; the drafter's engine is then cut over
        the same ranks (every rank builds one, `engine/follow.py` keeps them in step) while the fusion matrix and the
        fused features stay whole on every rank, as the tapped rows they are made from are."""
        self.window = int(window)
        self.ring = int(ring) if ring else 2 * self.window
        assert self.window == 0 or self.ring > self.window + block, "the ring must hold a window and a block"
        ecfg = EngineConfig(n_slots=n_slots, max_ctx=(self.ring + block + 2) if self.window else max_ctx, use_graphs=False,
                            weight_dtype=weight_dtype)
        self.eng = Engine(cfg, weights, ecfg, device=device, seed=seed, tp=tp)
        self.base = [0] * n_slots                    # target position of the drafter's local position 0
        self.hist = [[] for _ in range(n_slots)]     # windowed mode: (tokens, fused features or None) of recent commits
        self.block = block
        self.tree_k = 4                              # candidates per depth when growing a verify tree
        self.mask_token = mask_token
        g = torch.Generator().manual_seed(seed + 17)
        self.n_taps = n_taps
        self.fuse = (torch.randn(cfg.hidden, n_taps * target_hidden, generator=g) * 0.02).to(self.eng.device, self.eng.dtype)
        self.last_feat = [None] * n_slots            # fused features of the last committed row of each slot
        # rolling signature of the tokens held at the drafter's local positions 0 .. len - 1 of each slot: sig[i] covers
        # the first i tokens. A window snapshot is only rolled back to when the slot still holds the snapshot's tokens
        # (a snapshot restored into a slot that another conversation has used since finds other rows there)
        self.sigs = [[0] for _ in range(n_slots)]

    def _fused(self, taps, rows: slice) -> Optional[torch.Tensor]:
        if not taps or self.n_taps == 0:
            return None
        cat = torch.cat([t[rows].to(self.eng.device, self.eng.dtype) for t in taps[:self.n_taps]], -1)
        return (cat.float() @ self.fuse.float().t()).to(self.eng.dtype)

    def reset(self, slot: int) -> None:
        self.eng.reset_slot(slot)
        self.last_feat[slot] = None
        self.base[slot] = 0
        self.hist[slot] = []
        self.sigs[slot] = [0]

    _SIG_P, _SIG_M = 1000003, (1 << 61) - 1

    def _note(self, slot: int, local: int, tokens: Sequence[int]) -> None:
        """Tokens were written at the slot's local positions local .. local + n - 1."""
        sg = self.sigs[slot]
        del sg[local + 1:]
        if len(sg) != local + 1:                     # rows below `local` that this drafter never wrote: no valid signature
            sg[:] = [0] + [-1] * local
        for t in tokens:
            sg.append((sg[-1] * self._SIG_P + int(t) + 1) % self._SIG_M if sg[-1] >= 0 else -1)

    def _place(self, slot: int, pos0: int) -> int:
        """Local position of target position pos0 in the slot's cache (whole-context mode). An empty slot starts its own
        positions at pos0; a gap behind the rows it holds (a restore the drafter could not follow) starts it over."""
        if self.eng.slot_len[slot] == 0:
            self.base[slot] = pos0
        local = pos0 - self.base[slot]
        if local < 0 or local > self.eng.slot_len[slot]:
            self.eng.reset_slot(slot)
            self.sigs[slot] = [0]
            self.base[slot] = pos0
            local = 0
        return local

    def _hist_tokens(self, slot: int) -> int:
        return sum(len(t) for t, _ in self.hist[slot])

    def _hist_trim(self, slot: int, keep: int) -> None:
        """Keep only the last `keep` tokens of the slot's commit history."""
        h = self.hist[slot]
        extra = self._hist_tokens(slot) - keep
        while extra > 0 and h:
            t, f = h[0]
            if len(t) <= extra:
                h.pop(0)
                extra -= len(t)
            else:
                h[0] = (t[extra:], None if f is None else f[extra:])
                extra = 0

    def _hist_drop_tail(self, slot: int, k: int) -> None:
        h = self.hist[slot]
        while k > 0 and h:
            t, f = h[-1]
            if len(t) <= k:
                h.pop()
                k -= len(t)
            else:
                h[-1] = (t[:-k], None if f is None else f[:-k])
                k = 0

    def absorb(self, slot: int, tokens: Sequence[int], pos0: int, taps) -> None:
        """Extend the drafter's cache with committed tokens and the target features of their rows."""
        n = len(tokens)
        if n == 0:
            return
        feat = self._fused(taps, slice(0, n)) if taps and taps[0].shape[0] >= n else None
        local = pos0 if self.window else self._place(slot, pos0)
        if self.window and n > self.window:
            # a commit longer than the window (a prompt chunk): only its last `window` rows can matter afterwards
            cut = n - self.window
            tokens, pos0, n = list(tokens)[cut:], pos0 + cut, self.window
            feat = None if feat is None else feat[cut:]
            self.eng.reset_slot(slot)
            self.hist[slot] = []
        if self.window:
            if self.eng.slot_len[slot] == 0 and not self.hist[slot]:
                self.base[slot] = pos0                       # an empty drafter starts its own positions here
            local = pos0 - self.base[slot]
            if local < 0 or local + n > self.ring:
                # rebuild the slot from the last `window` committed tokens, then go on behind them
                self._hist_trim(slot, min(self.window, max(0, self.ring - n)))
                kept = [t for ts, _ in self.hist[slot] for t in ts]
                feats = [f for _, f in self.hist[slot]]
                self.eng.reset_slot(slot)
                self.base[slot] = pos0 - len(kept)
                self.sigs[slot] = [0]
                if kept:
                    x_add = torch.cat(feats) if all(f is not None for f in feats) else None
                    self.eng.forward([Segment(slot, 0, kept, "none")], commit=True, x_add=x_add)
                    self._note(slot, 0, kept)
                local = len(kept)
            self.hist[slot].append(([int(t) for t in tokens], None if feat is None else feat.clone()))
            self._hist_trim(slot, self.window)
        self.eng.forward([Segment(slot, local, list(tokens), "none")], commit=True, x_add=feat)
        self._note(slot, local, tokens)
        if feat is not None:
            self.last_feat[slot] = feat[-1:].clone()

    def draft(self, slot: int, last_token: int, pos: int, taps, n: int) -> List[int]:
        n = min(n, self.block)
        if n <= 0:
            return []
        toks = [last_token] + [self.mask_token] * (n - 1)
        feat = self.last_feat[slot]
        x_add = feat.expand(n, -1).contiguous() if feat is not None else None
        _, picks, _ = self.eng.forward([Segment(slot, pos - self.base[slot], toks, "all")], commit=False, greedy=True, x_add=x_add)
        return [int(t) for t in picks[0].tolist()]

    def draft_tree(self, slot: int, last_token: int, pos: int, taps, depth: int, rows: int):
        """One block pass scores every depth at once; the `tree_k` best tokens of each depth are grown into a
        best-first tree of `rows` draft rows (reference `draft_trees`, `crates/fe-dflash/src/lib.rs:841`)."""
        n = min(depth, self.block)
        if n <= 0 or rows <= 0:
            return [], []
        toks = [last_token] + [self.mask_token] * (n - 1)
        feat = self.last_feat[slot]
        x_add = feat.expand(n, -1).contiguous() if feat is not None else None
        logits, _, _ = self.eng.forward([Segment(slot, pos - self.base[slot], toks, "all")], commit=False, greedy=False, x_add=x_add)
        lp, ids = torch.log_softmax(logits.float(), -1).topk(min(self.tree_k, logits.shape[-1]), -1)
        lp, ids = lp.tolist(), ids.tolist()
        return grow_tree([list(zip(ids[d], lp[d])) for d in range(n)], rows)

    # ---- several requests of one step in one pass of the drafter --------------------------------------------------
    def _block_pass(self, reqs, greedy: bool):
        """One forward over [last token, MASK ...] blocks of several slots. reqs: (slot, last_token, pos, n) with n > 0.
        Returns the forward's (logits, picks) with the requests' rows back to back."""
        segs, adds = [], []
        any_feat = any(self.last_feat[slot] is not None for slot, _, _, _ in reqs)
        for slot, tok, pos, n in reqs:
            segs.append(Segment(slot, pos - self.base[slot], [tok] + [self.mask_token] * (n - 1), "all"))
            if any_feat:
                f = self.last_feat[slot]
                adds.append(f.expand(n, -1) if f is not None else
                            torch.zeros(n, self.eng.full_cfg.hidden, device=self.eng.device, dtype=self.eng.dtype))
        x_add = torch.cat(adds).contiguous() if any_feat else None
        logits, picks, _ = self.eng.forward(segs, commit=False, greedy=greedy, x_add=x_add)
        return logits, picks

    def draft_many(self, reqs, taps) -> List[List[int]]:
        live = [(i, slot, tok, pos, min(n, self.block)) for i, (slot, tok, pos, n) in enumerate(reqs) if min(n, self.block) > 0]
        out: List[List[int]] = [[] for _ in reqs]
        if len(live) == 1:
            i, slot, tok, pos, n = live[0]
            out[i] = self.draft(slot, tok, pos, taps, n)
        elif live:
            _, picks = self._block_pass([x[1:] for x in live], greedy=True)
            ids, r = picks[0].tolist(), 0
            for i, _, _, _, n in live:
                out[i] = [int(t) for t in ids[r:r + n]]
                r += n
        return out

    def draft_tree_many(self, reqs, taps):
        live = [(i, slot, tok, pos, min(depth, self.block), rows) for i, (slot, tok, pos, depth, rows) in enumerate(reqs)
                if min(depth, self.block) > 0 and rows > 0]
        out = [([], []) for _ in reqs]
        if len(live) == 1:
            i, slot, tok, pos, n, rows = live[0]
            out[i] = self.draft_tree(slot, tok, pos, taps, n, rows)
        elif live:
            logits, _ = self._block_pass([x[1:5] for x in live], greedy=False)
            lp, ids = torch.log_softmax(logits.float(), -1).topk(min(self.tree_k, logits.shape[-1]), -1)
            lp, ids, r = lp.tolist(), ids.tolist(), 0
            for i, _, _, _, n, rows in live:
                out[i] = grow_tree([list(zip(ids[r + d], lp[r + d])) for d in range(n)], rows)
                r += n
        return out

    def absorb_rows_many(self, items, taps) -> None:
        """Kept rows of several requests into the drafter's cache in one forward (whole-context mode; a bounded window
        keeps its per-slot path, whose rebuilds do not batch)."""
        from ..engine.scheduler import select_rows
        items = [it for it in items if len(it[1]) > 0]
        if self.window or len(items) <= 1 or not taps or self.n_taps == 0:
            for slot, tokens, pos0, rows in items:
                self.absorb_rows(slot, tokens, pos0, taps, rows)
            return
        segs, feats = [], []
        for slot, tokens, pos0, rows in items:
            sel = select_rows(taps, rows)
            n = len(tokens)
            if sel[0].shape[0] < n:                          # fewer tap rows than tokens: the per-slot path decides
                for it in items:
                    self.absorb_rows(it[0], it[1], it[2], taps, it[3])
                return
            feats.append(self._fused(sel, slice(0, n)))
            segs.append(Segment(slot, self._place(slot, pos0), [int(t) for t in tokens], "none"))
        self.eng.forward(segs, commit=True, x_add=torch.cat(feats).contiguous())
        for (slot, tokens, _, _), seg, f in zip(items, segs, feats):
            self._note(slot, seg.pos0, tokens)
            self.last_feat[slot] = f[-1:].clone()

    def save_window(self, slot: int):
        n = self.eng.slot_len[slot]
        sg = self.sigs[slot]
        return {"len": n, "feat": self.last_feat[slot], "base": self.base[slot], "sig": sg[n] if n < len(sg) else -1}

    def restore_window(self, slot: int, blob) -> None:
        # When the slot still holds the snapshot's rows (same local positions, same tokens: the signature tells), only
        # the length rolls back. A slot that was rebuilt since (windowed mode), or that another conversation has used
        # (a snapshot restored into another slot), does not hold them: the drafter starts over, empty, from the next
        # absorbed row.
        sg = self.sigs[slot]
        n = -1 if blob is None else int(blob["len"])
        if (blob is None or blob.get("base", 0) != self.base[slot] or n > self.eng.slot_len[slot] or n >= len(sg)
                or sg[n] < 0 or sg[n] != blob.get("sig", -1)):
            self.reset(slot)
            return
        cur = self.eng.slot_len[slot]
        self.eng.slot_len[slot] = n
        del sg[n + 1:]
        if self.window and cur > n:
            self._hist_drop_tail(slot, cur - n)
        self.last_feat[slot] = blob["feat"]


class OracleDrafter(Drafter):
    """A drafter whose acceptance rate is a dial: it proposes the tokens the target is known to produce (`truth`, recorded
    from a plain greedy run of the same prompt) and corrupts every proposed token with probability 1 - p (the first
    corrupted token ends what the verify step accepts). For benchmarks and tests of the speculative path: the cost of
    the step (verify rows, commit, replay) is real, the acceptance rate is chosen, and the output must equal the plain
    run's. With `cost_model` set (a `BlockDrafter`), its draft pass runs every step too, so the time of a real draft
    model is charged while the tokens come from the oracle."""

    def __init__(self, p: float, vocab: int, seed: int = 0, cost_model: Optional[Drafter] = None):
        self.p = float(p)
        self.vocab = vocab
        self.truth = {}                              # slot -> (position of truth[0], tokens)
        self.rng = torch.Generator().manual_seed(seed)
        self.cost_model = cost_model

    def set_truth(self, slot: int, pos0: int, tokens: Sequence[int]) -> None:
        self.truth[slot] = (int(pos0), [int(t) for t in tokens])

    def draft(self, slot: int, last_token: int, pos: int, taps, n: int) -> List[int]:
        if self.cost_model is not None:
            self.cost_model.draft(slot, last_token, pos, taps, n)
        return self._pick(slot, pos, n)

    def draft_many(self, reqs, taps) -> List[List[int]]:
        if self.cost_model is not None:
            self.cost_model.draft_many(reqs, taps)           # one pass of the real drafter for all requests, as in serving
        return [self._pick(slot, pos, n) for slot, _, pos, n in reqs]

    def absorb_rows_many(self, items, taps) -> None:
        if self.cost_model is not None:
            self.cost_model.absorb_rows_many(items, taps)

    def _pick(self, slot: int, pos: int, n: int) -> List[int]:
        if slot not in self.truth or n <= 0:
            return []
        pos0, toks = self.truth[slot]
        i = pos + 1 - pos0                           # the row at `pos` holds last_token; the draft starts one later
        out = [int(t) for t in toks[max(i, 0):max(i, 0) + n]]
        if not out:
            return []
        keep = torch.rand(len(out), generator=self.rng) < self.p
        for j in range(len(out)):
            if not bool(keep[j]):
                out[j] = (out[j] + 1 + int(torch.randint(0, self.vocab - 1, (1,), generator=self.rng))) % self.vocab
        return out

    def absorb(self, slot, tokens, pos0, taps):
        if self.cost_model is not None:
            self.cost_model.absorb(slot, tokens, pos0, taps)

    def reset(self, slot):
        if self.cost_model is not None:
            self.cost_model.reset(slot)
