"""Leader / follower control of tensor-parallel ranks: rank 0 runs the scheduler (and the HTTP server) and every call it
makes on its engine is replayed, in order, by the other ranks on theirs. The stream is a sequence of small pickled
records (method path, arguments) broadcast over a CPU-side control group, so the GPU collectives inside the calls stay
in lockstep without any rank but the leader deciding anything.

Counterpart of the reference's follower RPC (`crates/fe-model/src/follow.rs:1-306`: a 16-variant `Call` enum streamed
over TCP; `Engine::mirror` / `follow_with`, `crates/fe-model/src/model.rs:1606-1755`).

State snapshots are per-rank tensors, so they travel as integer handles: `ex.state_save` makes one on every rank under
the same id, `ex.state_restore` names it, and ids the leader's garbage collector has released ride along with the next
record so followers free theirs.

A draft model is mirrored one level up, at the `Drafter` interface (`Leader.attach_drafter`): every rank holds its own
drafter over its own shard of the draft engine, and the leader's `absorb_rows` / `draft` / `draft_tree` / `reset` /
`save_window` / `restore_window` calls are replayed as such. The target's tapped hidden rows never travel: they are
replicated by the target's own step, so a follower reads them from its engine and applies the row selection (plain
integers) the leader sent. The draft engine's collectives then run in the same order on every rank, between the
target's. The drafted tokens a follower computes are dropped; only the leader's scheduler decides.
"""
from __future__ import annotations

import weakref
from typing import Any, Dict, List

MIRRORED = {
    "forward", "commit_verified", "commit_tree", "reset_slot", "prefill",
    "ex.attach_blocks", "ex.copy_blocks", "ex.detach_blocks", "ex.ensure_capacity", "ex.pool.release",
    "ex.state_save", "ex.state_restore", "ex.copy_slot",
}


class SnapHandle:
    """Leader-side stand-in for a state snapshot: the local tensors plus the id the followers know it by."""

    def __init__(self, sid: int, local):
        self.sid, self.local = sid, local


class _Proxy:
    def __init__(self, leader: "Leader", target, path: str):
        object.__setattr__(self, "_l", leader)
        object.__setattr__(self, "_t", target)
        object.__setattr__(self, "_p", path)

    def __getattr__(self, name):
        leader, target, path = self._l, self._t, self._p
        full = f"{path}.{name}" if path else name
        attr = getattr(target, name)
        if full in MIRRORED:
            return lambda *a, **kw: leader.call(full, attr, a, kw)
        if any(m.startswith(full + ".") for m in MIRRORED):
            return _Proxy(leader, attr, full)
        return attr

    def __setattr__(self, name, value):
        setattr(self._t, name, value)


class Leader(_Proxy):
    """Wraps rank 0's engine: same attributes, mirrored methods are broadcast before they run locally."""

    def __init__(self, engine, tp):
        super().__init__(self, engine, "")
        object.__setattr__(self, "tp", tp)
        object.__setattr__(self, "_next_sid", 1)
        object.__setattr__(self, "_dropped", [])

    def call(self, path: str, fn, args, kwargs):
        if path == "forward":
            assert kwargs.get("x_add") is None and len(args) < 4, "feature injection is not mirrored"
        if path == "ex.state_restore":
            h = args[1]
            wire = (args[0], h.sid)
            self._send(path, wire, {})
            return fn(args[0], h.local)
        if path == "ex.state_save":
            sid = self.new_sid()
            self._send(path, args, {"_sid": sid})
            h = SnapHandle(sid, fn(*args, **kwargs))
            weakref.finalize(h, self._dropped.append, sid)
            return h
        self._send(path, args, kwargs)
        return fn(*args, **kwargs)

    def _send(self, path, args, kwargs):
        drops, self._dropped[:] = list(self._dropped), []
        self.tp.broadcast_object(("call", path, args, kwargs, drops))

    def new_sid(self) -> int:
        sid = self._next_sid
        object.__setattr__(self, "_next_sid", sid + 1)
        return sid

    def attach_drafter(self, drafter) -> "DrafterLeader":
        """Rank 0's draft model, mirrored: the followers were given theirs in `follow(engine, tp, drafter)`."""
        return DrafterLeader(self, drafter)

    def stop_followers(self) -> None:
        self.tp.broadcast_object(("stop",))


class DrafterLeader:
    """Rank 0's draft model under tensor parallelism: the `Drafter` interface, each call broadcast before it runs here."""

    def __init__(self, leader: Leader, drafter):
        self._l, self._d = leader, drafter

    def __getattr__(self, name):
        return getattr(self._d, name)

    def reset(self, slot: int) -> None:
        self._l._send("drafter.reset", (int(slot),), {})
        self._d.reset(slot)

    def absorb_rows(self, slot, tokens, pos0, taps, rows) -> None:
        rows = rows if rows is None or isinstance(rows, tuple) else [int(r) for r in rows]
        self._l._send("drafter.absorb_rows", (int(slot), [int(t) for t in tokens], int(pos0), rows), {})
        self._d.absorb_rows(slot, tokens, pos0, taps, rows)

    def absorb(self, slot, tokens, pos0, taps) -> None:
        raise TypeError("a mirrored drafter takes its rows by index: call absorb_rows")

    def draft(self, slot, last_token, pos, taps, n):
        self._l._send("drafter.draft", (int(slot), int(last_token), int(pos), int(n)), {})
        return self._d.draft(slot, last_token, pos, taps, n)

    def draft_tree(self, slot, last_token, pos, taps, depth, rows):
        self._l._send("drafter.draft_tree", (int(slot), int(last_token), int(pos), int(depth), int(rows)), {})
        return self._d.draft_tree(slot, last_token, pos, taps, depth, rows)

    def draft_many(self, reqs, taps):
        reqs = [tuple(int(v) for v in r) for r in reqs]
        self._l._send("drafter.draft_many", (reqs,), {})
        return self._d.draft_many(reqs, taps)

    def draft_tree_many(self, reqs, taps):
        reqs = [tuple(int(v) for v in r) for r in reqs]
        self._l._send("drafter.draft_tree_many", (reqs,), {})
        return self._d.draft_tree_many(reqs, taps)

    def absorb_rows_many(self, items, taps) -> None:
        items = [(int(slot), [int(t) for t in tokens], int(pos0),
                  rows if rows is None or isinstance(rows, tuple) else [int(r) for r in rows])
                 for slot, tokens, pos0, rows in items]
        self._l._send("drafter.absorb_rows_many", (items,), {})
        self._d.absorb_rows_many(items, taps)

    def save_window(self, slot):
        sid = self._l.new_sid()
        self._l._send("drafter.save_window", (int(slot),), {"_sid": sid})
        h = SnapHandle(sid, self._d.save_window(slot))
        weakref.finalize(h, self._l._dropped.append, sid)
        return h

    def restore_window(self, slot, blob) -> None:
        self._l._send("drafter.restore_window", (int(slot), None if blob is None else blob.sid), {})
        self._d.restore_window(slot, None if blob is None else blob.local)


def _replay_drafter(drafter, engine, name: str, args, kwargs, snaps) -> None:
    if drafter is None:
        raise RuntimeError("the leader mirrors a draft model and this rank was started without one")
    if name == "absorb_rows":
        slot, tokens, pos0, rows = args
        drafter.absorb_rows(slot, tokens, pos0, engine.taps, rows)
    elif name == "draft":
        slot, tok, pos, n = args
        drafter.draft(slot, tok, pos, engine.taps, n)
    elif name == "draft_tree":
        slot, tok, pos, depth, rows = args
        drafter.draft_tree(slot, tok, pos, engine.taps, depth, rows)
    elif name in ("draft_many", "draft_tree_many", "absorb_rows_many"):
        getattr(drafter, name)(args[0], engine.taps)
    elif name == "save_window":
        snaps[kwargs["_sid"]] = drafter.save_window(args[0])
    elif name == "restore_window":
        drafter.restore_window(args[0], None if args[1] is None else snaps[args[1]])
    elif name == "reset":
        drafter.reset(args[0])
    else:
        raise RuntimeError(f"unknown drafter call {name!r} in the leader's stream")


def follow(engine, tp, drafter=None) -> int:
    """Follower loop: replay the leader's calls until it says stop. Returns the number of calls replayed. `drafter`:
    this rank's draft model when the leader mirrors one (`Leader.attach_drafter`)."""
    snaps: Dict[int, Any] = {}
    n = 0
    while True:
        msg = tp.broadcast_object(None)
        if msg[0] == "stop":
            return n
        _, path, args, kwargs, drops = msg
        for sid in drops:
            snaps.pop(sid, None)
        if path.startswith("drafter."):
            _replay_drafter(drafter, engine, path.split(".", 1)[1], args, kwargs, snaps)
            n += 1
            continue
        target = engine
        parts: List[str] = path.split(".")
        for p in parts[:-1]:
            target = getattr(target, p)
        fn = getattr(target, parts[-1])
        if path == "ex.state_save":
            snaps[kwargs["_sid"]] = fn(*args)
        elif path == "ex.state_restore":
            fn(args[0], snaps[args[1]])
        else:
            fn(*args, **kwargs)
        n += 1
