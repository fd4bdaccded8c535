"""Leader / follower control of tensor-parallel ranks: rank 0 runs the scheduler (and the HTTP server) and every call it
makes on its engine is replayed, in order, by the other ranks on theirs. The stream is a sequence of small pickled
records (method path, arguments) broadcast over a CPU-side control group, so the GPU collectives inside the calls stay
in lockstep without any rank but the leader deciding anything.

Counterpart of the reference's follower RPC (`crates/fe-model/src/follow.rs:1-306`: a 16-variant `Call` enum streamed
over TCP; `Engine::mirror` / `follow_with`, `crates/fe-model/src/model.rs:1606-1755`).

State snapshots are per-rank tensors, so they travel as integer handles: `ex.state_save` makes one on every rank under
the same id, `ex.state_restore` names it, and ids the leader's garbage collector has released ride along with the next
record so followers free theirs.
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
            sid = self._next_sid
            object.__setattr__(self, "_next_sid", sid + 1)
            self._send(path, args, {"_sid": sid})
            h = SnapHandle(sid, fn(*args, **kwargs))
            weakref.finalize(h, self._dropped.append, sid)
            return h
        self._send(path, args, kwargs)
        return fn(*args, **kwargs)

    def _send(self, path, args, kwargs):
        drops, self._dropped[:] = list(self._dropped), []
        self.tp.broadcast_object(("call", path, args, kwargs, drops))

    def stop_followers(self) -> None:
        self.tp.broadcast_object(("stop",))


def follow(engine, tp) -> int:
    """Follower loop: replay the leader's calls until it says stop. Returns the number of calls replayed."""
    snaps: Dict[int, Any] = {}
    n = 0
    while True:
        msg = tp.broadcast_object(None)
        if msg[0] == "stop":
            return n
        _, path, args, kwargs, drops = msg
        for sid in drops:
            snaps.pop(sid, None)
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
