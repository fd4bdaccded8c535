"""Continuous-batching scheduler: admission with prompt-cache resume, decode / verify / prompt rows per step,
token selection, commit, snapshots, guards, failure bookkeeping.

Policy half of the reference's engine API (`crates/fe-model/src/sched.rs`: `Scheduler::start` `:253`, `submit` `:351`,
`Worker::run` `:802`, `admit_inner` `:952-1097`, `step` `:1099-1839`, `prompt_cut` `:636`, `tree_walk` `:125`,
`cache_save` `:1888`, `park_slot` `:1963`, `finish` `:2059`). Differences: no fixed cap of 4 requests (any number of
slots), paged KV so parking moves page ids instead of copying, and drafts are verified as chains.

One engine thread owns the device. `submit()` may be called from any thread; events go to the request's sink.
"""
from __future__ import annotations

import itertools
import os
import queue
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .copy import Copier, graft
from .engine import Engine, prompt_cuts
from .executor import Segment, TREE_MAX_ROWS
from .pcache import PREFIX_MIN, Park, SlotCache, Snap, common_prefix
from .sampler import Sampler, Sampling

STEP_FAILS_FATAL = 3      # consecutive failed steps that kill the engine (reference STEP_FAILS_FATAL)
DECODE_ROWS = 16          # most rows a request contributes to a verify segment (1 + drafts)


@dataclass
class SchedOptions:
    """Reference `SchedOptions` (`sched.rs:14-48`): FE_SPEC draft depth, FE_POOL park entries, FE_BATCH_ROWS."""

    spec: int = 0                      # draft tokens per step (0 = plain decoding)
    copy_rows: bool = True             # context-copy proposals
    copy_adaptive: bool = True         # their length follows how many of them land (doubling / halving between 4 and 64)
    pool: int = 64                     # parked entries kept
    batch_rows: int = 2048             # prompt rows per step
    finite_check: bool = True
    step_timeout_s: float = 120.0
    prof: int = 0                      # 1: one line per step on stderr; 2: verify steps add slots, rows fed and accepted paths
    share_min: int = PREFIX_MIN        # shortest common prefix worth waiting for / forking from a running request
    mixed: bool = True                 # decode rows and a prompt chunk share one forward when both are waiting
    tree_rows: int = 0                 # draft rows of a verify tree per request (0 = chains only; needs Drafter.draft_tree)
    device_sampling: bool = True       # plain sampled decode rows are drawn by the device sampler (no logits copy to the host)
    # FE_ARRIVAL_MS (0 = off): an idle engine woken by a request waits until no other has arrived for this long (at most
    # 4x in all, FE_ARRIVAL_MAX_MS while the server says more are coming), so requests sent together prefill in one forward
    arrival_ms: float = 5.0
    arrival_max_ms: float = 250.0
    # FE_DECODE_SHARE (0 = off): least fraction of wall time spent in decode-only steps while prompts are pending and some
    # stream decodes; FE_PREFILL_CAP: prompt rows a step may carry then (reference `sched.rs:513-528,1380-1392,1808-1818`)
    decode_share: float = 0.3
    prefill_cap: int = 2048

    @staticmethod
    def from_env() -> "SchedOptions":
        e = os.environ
        return SchedOptions(spec=int(e.get("FE_SPEC", "0")), pool=int(e.get("FE_POOL", "64")),
                            batch_rows=int(e.get("FE_BATCH_ROWS", "2048")),
                            finite_check=e.get("FE_FINITE_CHECK", "1") != "0",
                            step_timeout_s=float(e.get("FE_STEP_TIMEOUT", "120")), prof=int(e.get("FE_SCHED_PROF", "0")),
                            share_min=int(e.get("FE_SHARE_MIN", str(PREFIX_MIN))), tree_rows=int(e.get("FE_TREE", "0")),
                            arrival_ms=float(e.get("FE_ARRIVAL_MS", "5")), arrival_max_ms=float(e.get("FE_ARRIVAL_MAX_MS", "250")),
                            decode_share=min(0.95, max(0.0, float(e.get("FE_DECODE_SHARE", "0.3")))),
                            prefill_cap=max(4 * 32, int(e.get("FE_PREFILL_CAP", "2048"))))


@dataclass
class Event:
    kind: str                          # "tokens" | "finish" | "error"
    tokens: List[int] = field(default_factory=list)
    reason: str = ""                   # finish: "stop" | "length" | "cancelled" | "error" | "guard"
    timings: Dict[str, float] = field(default_factory=dict)
    message: str = ""


@dataclass
class Request:
    prompt: List[int]
    sampling: Sampling = field(default_factory=Sampling)
    sink: Optional[Callable[[Event], None]] = None
    snapshots: List[int] = field(default_factory=list)     # prompt positions worth a snapshot (template boundaries)
    cancel: threading.Event = field(default_factory=threading.Event)
    guard: Optional[Callable[[List[int]], Optional[str]]] = None   # called with new tokens; returns a finish reason
    rid: int = 0


@dataclass
class Active:
    req: Request
    slot: int
    pos: int                           # tokens whose state is in the slot
    pending: List[int]                 # prompt tokens not yet run
    sampler: Sampler
    copier: Optional[Copier]
    out: List[int] = field(default_factory=list)
    next_token: Optional[int] = None   # token to feed in the next decode row
    cached: int = 0                    # prompt tokens reused from the cache
    t_submit: float = 0.0
    t_first: float = 0.0
    t_prompt_done: float = 0.0
    drafts_proposed: int = 0
    drafts_accepted: int = 0
    snap_at: List[int] = field(default_factory=list)


def grow_tree(cands: Sequence[Sequence[Tuple[int, float]]], rows: int) -> Tuple[List[int], List[int]]:
    """Best-first verify tree from per-depth candidates. `cands[d]` lists (token, log-probability) for the draft
    token at depth d + 1 (a block drafter scores all depths in one pass, independently of the path taken). Nodes are
    added in order of their path's summed log-probability until `rows` draft rows exist. Returns (tokens, parents) of
    the draft rows in segment numbering: the root (the token being fed) is row 0, draft row i is row i + 1, parents
    come before children. Reference `grow_tree` (`crates/fe-dflash/src/lib.rs:306`)."""
    from .._ext import host
    h = host()
    if h is not None:                                        # C++ (`csrc/host_runtime.cpp`), the same heap discipline
        t2, p2 = h.host_grow_tree([[int(t) for t, _ in c] for c in cands], [[float(lp) for _, lp in c] for c in cands], int(rows))
        return list(t2), list(p2)
    import heapq
    toks: List[int] = []
    par: List[int] = []
    heap: List[Tuple[float, int, int, int, int]] = []       # (-score, tie, parent row, depth, candidate index)
    tie = 0
    if cands and cands[0]:
        heap.append((-float(cands[0][0][1]), tie, 0, 0, 0))
    while heap and len(toks) < rows:
        neg, _, prow, d, ci = heapq.heappop(heap)
        tok, lp = cands[d][ci]
        toks.append(int(tok))
        par.append(prow)
        me = len(toks)                                       # this node's row in the segment
        if ci + 1 < len(cands[d]):                           # next-best sibling under the same parent
            tie += 1
            heapq.heappush(heap, (neg + float(lp) - float(cands[d][ci + 1][1]), tie, prow, d, ci + 1))
        if d + 1 < len(cands) and cands[d + 1]:              # best child
            tie += 1
            heapq.heappush(heap, (neg - float(cands[d + 1][0][1]), tie, me, d + 1, 0))
    return toks, par


def tree_walk(tokens: Sequence[int], parents: Sequence[int], pick) -> Tuple[List[int], List[int]]:
    """Walk a verified tree from the root: `pick(row)` (a callable, or the list of all rows' picks) is the target's token
    after the row; descend into the child
    that carries it, stop when none does. Returns (rows of the accepted path, tokens to emit), one token per path
    row. Reference `tree_walk` (`crates/fe-model/src/sched.rs:125`)."""
    if not callable(pick):                                   # the picks as a list (greedy rows)
        from .._ext import host
        h = host()
        if h is not None:
            path, new = h.host_tree_walk([int(t) for t in tokens], [int(p) for p in parents], [int(t) for t in pick])
            return list(path), list(new)
        seq = pick
        pick = lambda node: seq[node]                        # noqa: E731
    kids: Dict[int, List[int]] = {}
    for r, p in enumerate(parents):
        if p >= 0:
            kids.setdefault(p, []).append(r)
    path, new, node = [0], [], 0
    while True:
        t = int(pick(node))
        new.append(t)
        nxt = next((c for c in kids.get(node, ()) if int(tokens[c]) == t), None)
        if nxt is None:
            return path, new
        path.append(nxt)
        node = nxt


def select_rows(taps, rows):
    """The rows of a step's tapped hidden states that a drafter is to read: all of them (`rows` None), a range
    `(start, stop)`, or a list of row indices (the accepted path of a verify tree)."""
    if rows is None or not taps:
        return taps
    if isinstance(rows, tuple):
        return [t[rows[0]:rows[1]] for t in taps]
    idx = torch.tensor([int(r) for r in rows], dtype=torch.long, device=taps[0].device)
    return [t.index_select(0, idx) for t in taps]


class Drafter:
    """Plug-in interface of a draft model (reference trait `Drafter`, `sched.rs:58-116`)."""

    def draft(self, slot: int, last_token: int, pos: int, taps, n: int) -> List[int]:
        return []

    def draft_tree(self, slot: int, last_token: int, pos: int, taps, depth: int, rows: int) -> Tuple[List[int], List[int]]:
        """Draft rows of a verify tree: (tokens, parents) in segment numbering (row 0 is `last_token`, draft row i is
        row i + 1). The default is the chain of `draft`."""
        d = self.draft(slot, last_token, pos, taps, min(depth, rows))
        return list(d), list(range(len(d)))

    def draft_many(self, reqs: Sequence[Tuple[int, int, int, int]], taps) -> List[List[int]]:
        """`draft` for several requests of one step, reqs[i] = (slot, last_token, pos, n). A draft model overrides this
        to run one pass for all of them; the default asks one by one."""
        return [self.draft(slot, tok, pos, taps, n) for slot, tok, pos, n in reqs]

    def draft_tree_many(self, reqs: Sequence[Tuple[int, int, int, int, int]], taps) -> List[Tuple[List[int], List[int]]]:
        """`draft_tree` for several requests, reqs[i] = (slot, last_token, pos, depth, rows)."""
        return [self.draft_tree(slot, tok, pos, taps, depth, rows) for slot, tok, pos, depth, rows in reqs]

    def absorb_rows_many(self, items: Sequence[Tuple[int, Sequence[int], int, object]], taps) -> None:
        """`absorb_rows` for several requests, items[i] = (slot, tokens, pos0, rows)."""
        for slot, tokens, pos0, rows in items:
            self.absorb_rows(slot, tokens, pos0, taps, rows)

    def absorb(self, slot: int, tokens: Sequence[int], pos0: int, taps) -> None:
        pass

    def absorb_rows(self, slot: int, tokens: Sequence[int], pos0: int, taps, rows) -> None:
        """`absorb` over a selection of the step's tap rows (`select_rows`). What the scheduler calls: the selection
        travels as plain integers, so a mirrored drafter can repeat it on every rank's own taps."""
        self.absorb(slot, tokens, pos0, select_rows(taps, rows))

    def reset(self, slot: int) -> None:
        pass

    def save_window(self, slot: int):
        return None

    def restore_window(self, slot: int, blob) -> None:
        pass


class Scheduler:
    def __init__(self, engine: Engine, opts: Optional[SchedOptions] = None, drafter: Optional[Drafter] = None):
        self.eng = engine
        self.opts = opts or SchedOptions()
        self.drafter = drafter
        n = engine.ecfg.n_slots
        self.free: List[int] = list(range(n))
        self.slot_cache: List[SlotCache] = [SlotCache() for _ in range(n)]
        self.active: Dict[int, Active] = {}
        self.waiting: "queue.Queue[Request]" = queue.Queue()
        self.backlog: List[Request] = []
        self.park = Park(self.opts.pool)
        self._ids = itertools.count(1)
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.dead_reason: Optional[str] = None
        self.step_no = 0
        self.fails = 0
        self.step_started = 0.0
        self.incoming = 0                 # requests the server is still preparing (arrival window; set by the adapter)
        self.t_pre = self.t_dec = 0.0     # decayed wall time of steps with / without prompt rows while a stream decodes
        self.clock = None                 # tests: a fake clock for the fairness bookkeeping (callable -> seconds)
        self.stats = {"steps": 0, "tokens": 0, "prompt_tokens": 0, "cached_tokens": 0, "drafted": 0, "accepted": 0}
        self.panic_step = int(os.environ.get("FE_TEST_PANIC_STEP", "0"))     # fault injection (host side only)
        self.eng.ex.reclaim = self._reclaim

    # ---- public ------------------------------------------------------------------------------------
    def submit(self, req: Request) -> int:
        req.rid = next(self._ids)
        self.waiting.put(req)
        return req.rid

    def start(self) -> None:
        self._thread = threading.Thread(target=self._run, name="ferrite-engine", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=10)

    def dead(self) -> Optional[str]:
        """Reason the engine is unusable: an unrecoverable step error, or a step running past the timeout."""
        if self.dead_reason:
            return self.dead_reason
        if self.step_started and time.time() - self.step_started > self.opts.step_timeout_s:
            return f"step {self.step_no} has been running for more than {self.opts.step_timeout_s:.0f} s"
        return None

    @property
    def running(self) -> int:
        return len(self.active)

    @property
    def queued(self) -> int:
        return self.waiting.qsize() + len(self.backlog)

    # ---- engine thread -----------------------------------------------------------------------------
    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                busy = self.run_once(block=True)
                if not busy:
                    continue
            except Exception as e:                                  # noqa: BLE001
                self.dead_reason = f"engine thread died: {e!r}"
                traceback.print_exc()
                for a in list(self.active.values()):
                    self._emit(a, Event("error", message=self.dead_reason))
                return

    def run_once(self, block: bool = False) -> bool:
        """Drain arrivals, admit, run one step. Returns False when idle. Tests drive the scheduler with this."""
        self._drain(block and not self.active and not self.backlog)
        self._admit()
        if not self.active:
            return False
        self.step_no += 1
        if self.panic_step and self.step_no == self.panic_step:
            raise RuntimeError("injected panic (FE_TEST_PANIC_STEP)")
        self.step_started = time.time()
        try:
            self._step()
            self.fails = 0
        except Exception as e:                                      # noqa: BLE001
            self.fails += 1
            if self.fails >= STEP_FAILS_FATAL:
                self.step_started = 0.0
                raise
            for a in list(self.active.values()):                    # fail the requests of this step, keep serving
                self._finish(a, "error", message=repr(e))
        self.step_started = 0.0
        self.stats["steps"] += 1
        return True

    def _drain(self, block: bool) -> None:
        try:
            if block:
                self.backlog.append(self.waiting.get(timeout=0.05))
                self._arrival_window()
            while True:
                self.backlog.append(self.waiting.get_nowait())
        except queue.Empty:
            pass

    def _arrival_window(self) -> None:
        """Woken from idle: give the requests sent together a moment to arrive, so they start in the same forward
        (reference `Worker::run` intake, `crates/fe-model/src/sched.rs:810-835`). `self.incoming` is the number of
        requests the server is still preparing (tokenising, rendering the template)."""
        w = self.opts.arrival_ms / 1e3
        if w <= 0:
            return
        t0 = time.time()
        cap, hard = t0 + 4 * w, t0 + self.opts.arrival_max_ms / 1e3
        while True:
            now = time.time()
            coming = self.incoming > 0 and now < hard
            left = min(w, (hard if coming else cap) - now)
            if left <= 0:
                break
            try:
                self.backlog.append(self.waiting.get(timeout=left))
            except queue.Empty:
                if not coming:
                    break

    # ---- admission ----------------------------------------------------------------------------------
    def _pick_slot(self, prompt: Sequence[int]) -> Optional[int]:
        """Free slot with the longest resumable prefix of this prompt (reference `admit_inner`)."""
        if not self.free:
            return None
        best, best_pos = self.free[0], -1
        for s in self.free:
            snap = self.slot_cache[s].best_snap(prompt)
            p = snap.pos if snap else (0 if self.slot_cache[s].tokens else -1)
            if p > best_pos:
                best, best_pos = s, p
        return best

    def _park_slot(self, slot: int) -> None:
        """Move a finished slot's pages and snapshots to the parked pool so the slot can take another sequence."""
        sc = self.slot_cache[slot]
        if sc.snaps:
            last = max(s.pos for s in sc.snaps)
            blocks = self.eng.ex.detach_blocks(slot, last)
            while len(self.park) >= self.opts.pool and self._reclaim():
                pass
            self.park.add(sc.tokens[:last], [s for s in sc.snaps if s.pos <= last], blocks)
        self.eng.reset_slot(slot)
        sc.clear()

    def _reclaim(self) -> bool:
        """Evict the least recently used parked sequence and return its pages to the pool."""
        ev = self.park.evict_lru()
        if ev is None:
            return False
        self.eng.ex.pool.release(ev.blocks)
        return True

    # ---- shared prefill: a request whose prompt starts like one that is being prefilled waits for it --------------
    def _share_point(self, prompt: Sequence[int], a: Active) -> int:
        """Position (on the prompt alignment grid) up to which `prompt` and the active request's prompt agree."""
        cp = min(common_prefix(a.req.prompt, prompt), len(prompt) - 1, len(a.req.prompt))
        align = self.eng.ecfg.prompt_align
        return cp // align * align

    def _should_wait(self, req: Request) -> bool:
        """True while an active request is still prefilling a long prefix this request shares: the leader gets a
        snapshot point there and the waiter is admitted once the leader has passed it, forking its state and pages
        instead of computing the prefix again (reference `share_point`, leader / waiter, `sched.rs:653`)."""
        for a in self.active.values():
            sp = self._share_point(req.prompt, a)
            if sp < self.opts.share_min or not a.pending or a.pos >= sp:
                continue
            if sp not in a.snap_at:
                a.snap_at = sorted(set(a.snap_at) | {sp})
            return True
        return False

    def _fork_source(self, prompt: Sequence[int]):
        """(active request, snapshot) with the longest snapshot inside the common prefix, or None."""
        best = None
        for a in self.active.values():
            snap = self.slot_cache[a.slot].best_snap(prompt)
            if snap is not None and snap.pos >= self.opts.share_min and (best is None or snap.pos > best[1].pos):
                best = (a, snap)
        return best

    def _admit(self) -> None:
        i = 0
        while i < len(self.backlog) and self.free:
            if self._should_wait(self.backlog[i]):
                i += 1
                continue
            req = self.backlog.pop(i)
            if req.cancel.is_set():
                if req.sink:
                    req.sink(Event("finish", reason="cancelled"))
                continue
            slot = self._pick_slot(req.prompt)
            self.free.remove(slot)
            sc = self.slot_cache[slot]
            snap = sc.best_snap(req.prompt)
            pe, ps = self.park.best(req.prompt)
            resume = 0
            fork = self._fork_source(req.prompt)
            if fork is not None and fork[1].pos > max(ps.pos if ps is not None else 0, snap.pos if snap is not None else 0):
                # fork from a running sequence: copy its pages up to the snapshot and take the snapshot's state
                src, fs = fork
                self._park_slot(slot) if sc.tokens else self.eng.reset_slot(slot)
                nb = (fs.pos + self.eng.ecfg.kv_block - 1) // self.eng.ecfg.kv_block
                self.eng.ex.ensure_capacity(slot, fs.pos)
                self.eng.ex.copy_blocks(self.eng.ex.slot_blocks[src.slot][:nb], self.eng.ex.slot_blocks[slot][:nb])
                self.eng.ex.state_restore(slot, fs.state["gdn"])
                if self.drafter:
                    self.drafter.restore_window(slot, fs.state.get("draft"))
                sc.tokens = list(self.slot_cache[src.slot].tokens[:fs.pos])
                sc.snaps = [x for x in self.slot_cache[src.slot].snaps if x.pos <= fs.pos]
                resume = fs.pos
                self.stats["forked"] = self.stats.get("forked", 0) + 1
            elif ps is not None and (snap is None or ps.pos > snap.pos):
                # restore a parked sequence into this slot: move (exclusive) or copy (shared) its pages
                if not pe.shared:
                    self.park.take(pe)                 # out of the pool first, so parking this slot cannot evict it
                self._park_slot(slot) if sc.tokens else self.eng.reset_slot(slot)
                nb = (ps.pos + self.eng.ecfg.kv_block - 1) // self.eng.ecfg.kv_block
                if pe.shared:
                    self.eng.ex.ensure_capacity(slot, ps.pos)
                    self.eng.ex.copy_blocks(pe.blocks[:nb], self.eng.ex.slot_blocks[slot][:nb])
                    self.park.touch(pe)
                else:
                    self.eng.ex.attach_blocks(slot, pe.blocks[:nb])
                    self.eng.ex.pool.release(pe.blocks[nb:])
                self.eng.ex.state_restore(slot, ps.state["gdn"])
                if self.drafter:
                    self.drafter.restore_window(slot, ps.state.get("draft"))
                sc.tokens, sc.snaps = list(pe.tokens[:ps.pos]), [s for s in pe.snaps if s.pos <= ps.pos]
                resume = ps.pos
            elif snap is not None:
                self.eng.ex.state_restore(slot, snap.state["gdn"])
                if self.drafter:
                    self.drafter.restore_window(slot, snap.state.get("draft"))
                sc.truncate(snap.pos)
                resume = snap.pos
            else:
                if sc.tokens:
                    self._park_slot(slot)
                else:
                    self.eng.reset_slot(slot)
                if self.drafter:
                    self.drafter.reset(slot)
            self.eng.slot_len[slot] = resume
            a = Active(req, slot, resume, list(req.prompt[resume:]), Sampler(req.sampling, request_seed=req.rid, prompt=req.prompt),
                       Copier() if (self.opts.copy_rows and self.opts.spec > 0) else None, cached=resume,
                       t_submit=time.time(), snap_at=sorted(p for p in req.snapshots if resume < p <= len(req.prompt)))
            self.active[slot] = a
            self.stats["cached_tokens"] += resume

    # ---- one step -----------------------------------------------------------------------------------
    def _step(self) -> None:
        t0 = time.time()
        self._step_clock0 = self.clock() if self.clock is not None else 0.0
        for a in list(self.active.values()):
            if a.req.cancel.is_set():
                self._finish(a, "cancelled")
        decoders = [a for a in self.active.values() if not a.pending and a.next_token is not None]
        prefills = [a for a in self.active.values() if a.pending]
        n_dec = n_pre = 0
        budget = self.opts.batch_rows
        # fairness: while streams decode, prompt chunks are capped and only get (1 - share) of the wall time
        decoding = bool(decoders)
        if not decoding:
            self.t_pre = self.t_dec = 0.0
        elif self.opts.decode_share > 0 and prefills:
            budget = min(budget, self.opts.prefill_cap)
            if self.t_pre * self.opts.decode_share > (1.0 - self.opts.decode_share) * self.t_dec:
                prefills = []                                       # a decode-only step
                self.stats["decode_only_steps"] = self.stats.get("decode_only_steps", 0) + 1
        if (decoders and prefills and self.opts.mixed and self.opts.spec == 0 and self.drafter is None
                and all(a.req.sampling.greedy for a in decoders)):
            # continuous batching: the decode rows ride along with a prompt chunk, one pass over the weights for both
            n_dec, n_pre = self._mixed_step(decoders, prefills[0], budget)
            budget -= n_pre
            prefills = prefills[1:]
        elif decoders:
            n_dec = self._decode_step(decoders)
        if prefills and budget > 0:
            n_pre += self._group_prefill(prefills, budget)
        if decoding and self.opts.decode_share > 0:
            dt = (self.clock() - self._step_clock0) if self.clock is not None else time.time() - t0
            self.t_pre *= 0.97                                      # decay: the share tracks the last few seconds
            self.t_dec *= 0.97
            if n_pre > 0:
                self.t_pre += dt
            else:
                self.t_dec += dt
        if self.opts.prof:
            import sys
            tail = ""
            lv = getattr(self, "_last_verify", None)
            if self.opts.prof >= 2 and lv is not None:
                import json
                tail = f" | slots {json.dumps(lv['slots'])} rows {json.dumps(lv['rows'])} paths {json.dumps(lv['paths'])}"
                self._last_verify = None
            print(f"step {self.step_no}: dec {n_dec} rows, prompt {n_pre} rows, {1e3 * (time.time() - t0):.2f} ms{tail}",
                  file=sys.stderr)

    def _prefill_cut(self, a: Active, budget: int):
        """Next chunk of a prompt: (rows, tokens, is the last chunk, greedy pick usable). Chunks end at snapshot
        positions so the state can be saved there."""
        cut = prompt_cuts(len(a.pending), min(self.eng.ecfg.prefill_chunk, max(32, budget)), self.eng.ecfg.prompt_align)[0]
        for sp in a.snap_at:
            if a.pos < sp < a.pos + cut:
                cut = sp - a.pos
                break
        last = cut == len(a.pending)
        greedy = a.req.sampling.greedy and not (a.req.sampling.banned_first and not a.out)
        return cut, a.pending[:cut], last, greedy

    def _mixed_step(self, decoders: List[Active], a: Active, budget: int):
        """One forward over a decode row of every decoding request plus the next prompt chunk of `a`."""
        cut, toks, last, greedy = self._prefill_cut(a, max(32, budget - len(decoders)))
        if not greedy:
            return self._decode_step(decoders), self._prefill_step(a, budget)
        segs = [Segment(d.slot, d.pos, [d.next_token], "last") for d in decoders]
        segs.append(Segment(a.slot, a.pos, toks, "last" if last else "none"))
        logits, picks, rows = self.eng.forward(segs, commit=True, greedy=True)
        ids = picks[0].tolist()
        if self.opts.finite_check and not bool(picks[1].all()):
            for d in decoders + [a]:
                self._finish(d, "error", message="non-finite logits")
            return len(decoders), cut
        for i, d in enumerate(decoders):
            d.pos += 1
            self._accept(d, [int(ids[i])])
        self._prefill_done(a, cut, toks, last, int(ids[len(decoders)]) if last else None)
        return len(decoders), cut

    def _group_prefill(self, prefills: List[Active], budget: int) -> int:
        """Prompt chunks of several requests in ONE forward (reference `group_prefill`,
        `crates/fe-model/src/model.rs:2279`): short remainders first, each request contributes its next chunk until the
        step's row budget is used, so four 2K prompts arriving together cost one pass over the weights, not four."""
        budget = min(budget, self.eng.ecfg.max_step_rows)
        if len(prefills) == 1:
            return self._prefill_step(prefills[0], budget)
        group = []
        for a in sorted(prefills, key=lambda a: len(a.pending)):
            if budget < 32 and group:
                break
            cut, toks, last, greedy = self._prefill_cut(a, budget)
            if cut > budget and group:
                continue
            group.append((a, cut, toks, last, greedy))
            budget -= cut
        if len(group) == 1:
            return self._prefill_step(group[0][0], group[0][1])
        segs = [Segment(a.slot, a.pos, toks, "last" if last else "none") for a, _, toks, last, _ in group]
        all_greedy = all(g for _, _, _, last, g in group if last)
        logits, picks, _ = self.eng.forward(segs, greedy=all_greedy)
        ids = picks[0].tolist() if (all_greedy and picks is not None) else None
        k = r = n = 0
        for a, cut, toks, last, _ in group:
            tok = None
            if last:
                # (a greedy step under tensor parallelism merges (max, index) pairs over the ranks and has no logits)
                finite_k = bool(picks[1][k]) if (ids is not None and logits is None) else bool(torch.isfinite(logits[k]).all())
                if self.opts.finite_check and not finite_k:
                    a.pos += cut
                    a.pending = a.pending[cut:]
                    self._finish(a, "error", message="non-finite logits")
                    k += 1
                    r += cut
                    continue
                tok = int(ids[k]) if ids is not None else a.sampler.sample(logits[k], first=not a.out)
                k += 1
            self._prefill_done(a, cut, toks, last, tok, (r, r + cut))
            r += cut
            n += cut
        return n

    def _prefill_step(self, a: Active, budget: int) -> int:
        """Run the next chunk of a prompt on its own."""
        cut, toks, last, greedy = self._prefill_cut(a, budget)
        logits, picks, _ = self.eng.forward([Segment(a.slot, a.pos, toks, "last" if last else "none")], greedy=greedy)
        tok = None
        if last:
            tok = int(picks[0][0]) if greedy else a.sampler.sample(logits[0], first=not a.out)
            finite = bool(picks[1][0]) if (greedy and logits is None) else bool(torch.isfinite(logits[0]).all())
            if self.opts.finite_check and not finite:
                a.pos += cut
                a.pending = a.pending[cut:]
                self._finish(a, "error", message="non-finite logits")
                return cut
        self._prefill_done(a, cut, toks, last, tok)
        return cut

    def _prefill_done(self, a: Active, cut: int, toks: List[int], last: bool, tok, tap_rows=None) -> None:
        a.pos += cut
        a.pending = a.pending[cut:]
        self.slot_cache[a.slot].tokens = (a.req.prompt + a.out)[:a.pos]
        self.stats["prompt_tokens"] += cut
        if self.drafter:
            # before the snapshot: the drafter window saved with it must end at the snapshot's position
            self.drafter.absorb_rows(a.slot, toks, a.pos - cut, self.eng.taps, tap_rows)
        if a.pos in a.snap_at:
            self._snapshot(a, pinned=(a.pos == a.snap_at[0]))
        if last:
            a.t_prompt_done = time.time()
            self._accept(a, [tok])

    def _decode_step(self, decoders: List[Active]) -> int:
        """One decode / verify step over all decoding requests: a row per request plus its draft rows."""
        segs, drafts, trees, copies = [], [], [], []
        # pass 1: every request's room and copy proposal; what the draft model is asked for is collected, so that it
        # drafts for all requests in one pass of its own (reference `draft_many` / `draft_trees`, `sched.rs:58-116`)
        rooms: List[int] = []
        want_tree: List[Tuple[int, int, int, int, int]] = []          # (slot, last token, position, depth, rows)
        want_chain: List[Tuple[int, int, int, int]] = []              # (slot, last token, position, n)
        ask: List[Optional[Tuple[str, int]]] = []                     # per request: ("tree" | "chain", index into its list)
        for a in decoders:
            room, copy, what = 0, [], None
            if self.opts.spec > 0:
                room = min(self.opts.spec, DECODE_ROWS - 1, a.req.sampling.max_tokens - len(a.out) - 1,
                           self.eng.ecfg.max_ctx - a.pos - 2)
                if room > 0:
                    if a.copier is not None:
                        a.copier.sync(a.req.prompt + a.out[:-1] + [a.next_token])
                        copy = a.copier.propose(room, adaptive=self.opts.copy_adaptive)
                    if self.drafter is not None and self.opts.tree_rows > 0:
                        n_rows = min(self.opts.tree_rows, TREE_MAX_ROWS - 1, self.eng.ecfg.max_ctx - a.pos - 2)
                        what = ("tree", len(want_tree))
                        want_tree.append((a.slot, a.next_token, a.pos, room, n_rows))
                    elif not copy and self.drafter is not None:
                        what = ("chain", len(want_chain))
                        want_chain.append((a.slot, a.next_token, a.pos, room))
            rooms.append(room)
            copies.append(copy)
            ask.append(what)
        got_tree = self.drafter.draft_tree_many(want_tree, self.eng.taps) if want_tree else []
        got_chain = self.drafter.draft_many(want_chain, self.eng.taps) if want_chain else []
        # pass 2: the rows of every request
        for a, room, copy, what in zip(decoders, rooms, list(copies), ask):
            d: List[int] = []
            par: Optional[List[int]] = None
            if what is not None and what[0] == "tree":
                # the draft model's tree, with the copy proposal grafted onto it: rows the tree already holds are
                # shared, the rest of the copy hangs below them as a chain (reference `graft`)
                n_rows = want_tree[what[1]][4]
                d, dp = got_tree[what[1]]
                toks, pars = [a.next_token] + [int(t) for t in d[:n_rows]], [-1] + [int(p) for p in dp[:n_rows]]
                if copy:
                    graft(toks, pars, copy, TREE_MAX_ROWS - len(toks))
                d = toks[1:]
                if d and pars[1:] != list(range(len(d))):
                    par = pars
            elif copy:
                d = copy
            elif what is not None:
                d = got_chain[what[1]]
            d = [int(t) for t in (d if par is not None else d[:room])]
            copies[len(drafts)] = copy if (par is not None or d[:len(copy)] == copy) else []
            drafts.append(d)
            trees.append(par)
            segs.append(Segment(a.slot, a.pos, [a.next_token] + d, "all", parents=par))
        spec = any(drafts)
        all_greedy = all(a.req.sampling.greedy for a in decoders)
        logits, picks, rows = self.eng.forward(segs, commit=not spec, greedy=all_greedy)
        ids = picks[0].tolist() if all_greedy else None
        if self.opts.finite_check:
            finite = bool(picks[1].all()) if all_greedy else bool(torch.isfinite(logits).all())
            if not finite:
                for a in decoders:
                    self._finish(a, "error", message="non-finite logits")
                return len(rows)
        keep, paths, r = [], [], 0
        absorbs: List[Tuple[int, List[int], int, object]] = []        # (slot, tokens fed, first position, tap rows)
        accepts: List[Tuple[Active, List[int]]] = []
        taps = self.eng.taps
        any_tree = any(t is not None for t in trees)
        dev_ids = None
        if (not spec and not all_greedy and self.opts.device_sampling and self.eng.device.type == "cuda"
                and hasattr(self.eng.ops, "sample")
                and all((not a.req.sampling.greedy) and a.req.sampling.presence_penalty == 0
                        and a.req.sampling.frequency_penalty == 0 and a.req.sampling.repetition_penalty == 1.0
                        for a in decoders)):
            # one draw per row on the device (top-k / top-p / min-p as on the host); the per-step seed comes from the
            # request's own generator, so a seeded request repeats. Penalties and drafts keep the host sampler.
            seeds = [a.sampler.rng.next_u64() for a in decoders]
            dev_ids = self.eng.ops.sample(logits, [a.req.sampling for a in decoders], seeds).tolist()
        for a, d, par, copy in zip(decoders, drafts, trees, copies):
            n = 1 + len(d)
            if par is not None:
                # verify tree: follow the target's choices from the root (reference `tree_walk`); sampling from the
                # target at every node and descending only on a match keeps the output distribution the target's
                def pick(node, a=a, r=r):
                    if all_greedy:
                        return int(ids[r + node])
                    t = a.sampler.sample(logits[r + node])
                    a.sampler.observe(t)
                    return t
                # greedy: the target's picks of all rows are known, the walk runs in C++ when the extension is built
                path, new = tree_walk([a.next_token] + d, par,
                                      [int(t) for t in ids[r:r + 1 + len(d)]] if all_greedy else pick)
                cut = self._stop_cut(a, new)
                path, new = path[:cut], new[:cut]
                paths.append(path)
                keep.append(len(new))
                acc = len(new) - 1
                a.drafts_proposed += len(d)
                a.drafts_accepted += acc
                self.stats["drafted"] += len(d)
                self.stats["accepted"] += acc
                fed = [a.next_token] + [d[i - 1] for i in path[1:]]
                if a.copier is not None and copy:
                    landed = next((j for j, (x, y) in enumerate(zip(fed[1:], copy)) if x != y), min(len(fed) - 1, len(copy)))
                    a.copier.observe(len(copy), landed)
                a.pos += len(new)
                absorbs.append((a.slot, fed, a.pos - len(new), [r + i for i in path]))
                accepts.append((a, new))
                r += n
                continue
            if all_greedy:
                # accept-while-match walk over the chain (reference `tree_walk` on a path)
                new = []
                for i in range(n):
                    t = int(ids[r + i])
                    new.append(t)
                    if i < len(d) and t != d[i]:
                        break
            elif dev_ids is not None:
                new = [int(dev_ids[r])]
                a.sampler.observe(new[0])
            else:
                new = a.sampler.spec_accept(logits[r:r + n], d)
            new = new[:self._stop_cut(a, new)]
            acc = len(new) - 1
            keep.append(len(new))
            paths.append(list(range(len(new))))
            a.drafts_proposed += len(d)
            a.drafts_accepted += acc
            self.stats["drafted"] += len(d)
            self.stats["accepted"] += acc
            if a.copier is not None and copy:
                a.copier.observe(len(copy), min(acc, len(copy)))
            fed = [a.next_token] + d[:acc]
            a.pos += len(new)
            absorbs.append((a.slot, fed, a.pos - len(new), (r, r + len(new))))
            accepts.append((a, new))
            r += n
        # the draft model takes the kept rows of all requests in one pass; the target's state advances along the kept
        # rows; only then are the tokens handed out: a request that ends here snapshots its slot for the next turn,
        # and that snapshot must hold the committed state and the drafter's absorbed rows
        if self.drafter is not None:
            self.drafter.absorb_rows_many(absorbs, taps)
        if spec and any_tree:
            self.eng.commit_tree(paths)
        elif spec:
            self.eng.commit_verified(keep)
        for a, new in accepts:
            self._accept(a, new, sampled=not all_greedy)
        if self.opts.prof >= 2 and spec:
            # per request of this verify step: slot, rows fed (1 + drafts) and the accepted path's row indices; what
            # `tools/sched_budget.py` replays under smaller draft budgets
            self._last_verify = {"slots": [a.slot for a in decoders], "rows": [1 + len(d) for d in drafts], "paths": paths}
        return len(rows)

    @staticmethod
    def _stop_cut(a: Active, new: List[int]) -> int:
        """How many of a verify step's accepted tokens count: up to and including the first stop token. Rows behind it
        are not committed, so the slot ends where the reply ends and its end-of-reply snapshot serves the next turn."""
        stops = a.req.sampling.stop_ids
        if stops:
            for i, t in enumerate(new):
                if t in stops:
                    return i + 1
        return len(new)

    # ---- bookkeeping --------------------------------------------------------------------------------
    def _snapshot(self, a: Active, pinned: bool = False) -> None:
        state = {"gdn": self.eng.ex.state_save(a.slot)}
        if self.drafter:
            state["draft"] = self.drafter.save_window(a.slot)
        self.slot_cache[a.slot].push(Snap(a.pos, state, pinned))

    def _accept(self, a: Active, toks: List[int], sampled: bool = False) -> None:
        """Record newly chosen tokens: emit them, detect stop / length / guard, set the next input token."""
        if a.slot not in self.active:
            return
        if not a.t_first:
            a.t_first = time.time()
        emit: List[int] = []
        reason = None
        for t in toks:
            if not sampled:
                a.sampler.observe(t)                  # (speculative sampling already counted its own tokens)
            if t in a.req.sampling.stop_ids:
                reason = "stop"
                break
            emit.append(t)
            a.out.append(t)
            if len(a.out) >= a.req.sampling.max_tokens:
                reason = "length"
                break
        if emit:
            self.stats["tokens"] += len(emit)
            self._emit(a, Event("tokens", tokens=emit))
            if a.req.guard is not None and reason is None:
                g = a.req.guard(emit)
                if isinstance(g, (list, tuple)) and g:
                    # forced continuation (e.g. the closing tag of a capped reasoning block): the tokens become part
                    # of the reply and are run through the slot like prompt rows before sampling resumes
                    forced = [int(t) for t in g]
                    a.out.extend(forced)
                    self._emit(a, Event("tokens", tokens=forced))
                    a.pending = [toks[-1]] + forced
                    a.next_token = None
                    return
                if g:
                    reason = g
        if reason:
            self._finish(a, reason)
        else:
            a.next_token = toks[-1]
            self.slot_cache[a.slot].tokens = a.req.prompt + a.out[:-1]

    def _emit(self, a: Active, ev: Event) -> None:
        if a.req.sink:
            try:
                a.req.sink(ev)
            except Exception:                                       # a closed stream cancels the request
                a.req.cancel.set()

    def _finish(self, a: Active, reason: str, message: str = "") -> None:
        if a.slot not in self.active:
            return
        now = time.time()
        timings = {
            "prompt_n": len(a.req.prompt) - a.cached, "cache_n": a.cached,
            "prompt_ms": 1e3 * ((a.t_prompt_done or now) - a.t_submit),
            "predicted_n": len(a.out), "predicted_ms": 1e3 * (now - (a.t_prompt_done or now)),
            "draft_n": a.drafts_proposed, "draft_accepted_n": a.drafts_accepted,
        }
        # the slot keeps its sequence for a later turn; a snapshot at the end of the reply makes it resumable
        if reason in ("stop", "length") and a.next_token is not None:
            sc = self.slot_cache[a.slot]
            sc.tokens = (a.req.prompt + a.out)[:a.pos]
            self._snapshot(a)
        del self.active[a.slot]
        self.free.append(a.slot)
        kind = "error" if reason == "error" else "finish"
        self._emit(a, Event(kind, reason=reason, timings=timings, message=message))


def generate(sched: Scheduler, prompts: Sequence[Sequence[int]], sampling: Optional[Sampling] = None,
             snapshots: Optional[Sequence[Sequence[int]]] = None) -> List[List[int]]:
    """Synchronous helper: run prompts to completion through the scheduler (single-threaded stepping)."""
    outs: List[List[int]] = [[] for _ in prompts]
    done = [False] * len(prompts)
    errors: List[str] = []

    def sink(i):
        def f(ev: Event):
            if ev.kind == "tokens":
                outs[i].extend(ev.tokens)
            else:
                done[i] = True
                if ev.kind == "error":
                    errors.append(f"prompt {i}: {ev.message}")
        return f

    for i, p in enumerate(prompts):
        smp = sampling[i] if isinstance(sampling, (list, tuple)) else sampling      # one Sampling, or one per prompt
        sched.submit(Request(list(p), smp or Sampling(), sink(i),
                             snapshots=list(snapshots[i]) if snapshots else []))
    guard = 0
    while not all(done):
        sched.run_once()
        guard += 1
        assert guard < 100000, "scheduler made no progress"
    if errors:                                       # a helper for tests and benchmarks: a failed request is a failure
        raise RuntimeError("; ".join(errors))
    return outs
