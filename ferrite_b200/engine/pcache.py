"""Turn-boundary prompt cache: per-slot snapshots, the parked-sequence pool and shared-prefix lookup.

Data structures of the reference's `crates/fe-model/src/pcache.rs` (`Snap`, `KEEP_LAST` 2, `best_snap`, `truncate`,
`push`, `Park::{best, evict_lru, has_prefix}`) and the policy constants of `sched.rs:596-630`. A hybrid model can
only be resumed where its Gated DeltaNet state was saved: KV rows up to any position stay valid in the slot, but
the recurrent + conv state exists only at snapshot positions, so a resume point is always a snapshot position.

With a paged KV cache a parked sequence is a list of page ids handed over by the slot (no copy); restoring it
into a free slot either moves the pages back (exclusive entry) or copies them (an entry kept for other sessions,
e.g. a shared system prompt).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

KEEP_LAST = 2          # snapshots kept per slot besides the pinned first one
PREFIX_MIN = 1024      # shortest common prefix worth a shared-prefix entry
SHARE_NEAR = 256       # requests arriving together share a prefill when their common prefix is this long
SHARE_MAX = 4


def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    """Length of the common prefix. Unrelated sequences differ in their first tokens and leave at once; a matching history
    of 100K tokens is compared slice by slice (list equality runs in C) with doubling steps, and the slice that differs is
    bisected: a few hundred interpreter steps instead of one per token, at every admission, for every slot and parked entry."""
    n = min(len(a), len(b))
    if n == 0 or a[0] != b[0]:
        return 0
    if type(a) is not type(b) or not isinstance(a, (list, tuple)):
        a, b = list(a), list(b)              # slices of different sequence types never compare equal
    lo, step = 0, 64
    hi = n
    while lo < n:
        hi = min(n, lo + step)
        if a[lo:hi] == b[lo:hi]:
            lo, step = hi, step * 2
        else:
            break
    else:
        return n
    while hi - lo > 16:                      # a[:lo] == b[:lo], and a[lo:hi] != b[lo:hi]
        mid = (lo + hi) // 2
        if a[lo:mid] == b[lo:mid]:
            lo = mid
        else:
            hi = mid
    while lo < hi and a[lo] == b[lo]:
        lo += 1
    return lo


@dataclass
class Snap:
    pos: int                   # tokens consumed when the state was saved
    state: Any                 # engine-specific state blob (GDN rec + conv state, drafter window)
    pinned: bool = False       # system-prompt boundary: survives KEEP_LAST trimming


@dataclass
class SlotCache:
    """What a slot remembers between requests: its token history and the snapshots taken along it."""

    tokens: List[int] = field(default_factory=list)
    snaps: List[Snap] = field(default_factory=list)

    def push(self, snap: Snap) -> None:
        self.snaps = [s for s in self.snaps if s.pos != snap.pos]
        self.snaps.append(snap)
        self.snaps.sort(key=lambda s: s.pos)
        loose = [s for s in self.snaps if not s.pinned]
        for s in loose[:-KEEP_LAST] if len(loose) > KEEP_LAST else []:
            self.snaps.remove(s)

    def truncate(self, pos: int) -> None:
        """Forget everything after pos (the sequence was rolled back to a snapshot)."""
        self.tokens = self.tokens[:pos]
        self.snaps = [s for s in self.snaps if s.pos <= pos]

    def best_snap(self, prompt: Sequence[int]) -> Optional[Snap]:
        """Latest snapshot inside the common prefix of the slot's history and the new prompt. The prompt must
        keep at least one token to run, so a snapshot at len(prompt) is not usable."""
        cp = common_prefix(self.tokens, prompt)
        best = None
        for s in self.snaps:
            if s.pos <= cp and s.pos < len(prompt) and (best is None or s.pos > best.pos):
                best = s
        return best

    def clear(self) -> None:
        self.tokens, self.snaps = [], []


@dataclass
class ParkEntry:
    key: int
    tokens: List[int]
    snaps: List[Snap]
    blocks: List[int]          # KV pages covering len(tokens)
    shared: bool = False       # kept after a restore (pages are copied out instead of moved)
    last_use: int = 0


class Park:
    """LRU pool of parked sequences (reference `park_slot` `sched.rs:1963`, `park_restore` `:1983`)."""

    def __init__(self, max_entries: int = 64):
        self.entries: Dict[int, ParkEntry] = {}
        self.max_entries = max_entries
        self._ids = itertools.count(1)
        self._clock = itertools.count(1)

    def add(self, tokens: List[int], snaps: List[Snap], blocks: List[int], shared: bool = False) -> ParkEntry:
        e = ParkEntry(next(self._ids), list(tokens), list(snaps), list(blocks), shared, next(self._clock))
        self.entries[e.key] = e
        return e

    def best(self, prompt: Sequence[int]) -> Tuple[Optional[ParkEntry], Optional[Snap]]:
        """Entry and snapshot giving the longest resumable prefix of `prompt`."""
        best_e, best_s = None, None
        for e in self.entries.values():
            cp = common_prefix(e.tokens, prompt)
            for s in e.snaps:
                if s.pos <= cp and s.pos < len(prompt) and (best_s is None or s.pos > best_s.pos):
                    best_e, best_s = e, s
        return best_e, best_s

    def has_prefix(self, prompt: Sequence[int], min_len: int = PREFIX_MIN) -> bool:
        e, s = self.best(prompt)
        return s is not None and s.pos >= min_len

    def touch(self, e: ParkEntry) -> None:
        e.last_use = next(self._clock)

    def take(self, e: ParkEntry) -> ParkEntry:
        return self.entries.pop(e.key)

    def evict_lru(self) -> Optional[ParkEntry]:
        if not self.entries:
            return None
        e = min(self.entries.values(), key=lambda x: (x.shared, x.last_use))
        return self.entries.pop(e.key)

    def __len__(self) -> int:
        return len(self.entries)
