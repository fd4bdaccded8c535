"""Bounds-checked debug mode: every index tensor an op receives is checked on the host before the kernel runs.

The kernels trust their tables (slot ids, page ids, positions, token ids, expert ids): an index out of range is a read or
write outside an allocation, which on the GPU is at best silent corruption. Attached to an engine, this proxy looks at the
arguments of every op call by parameter name, checks each index tensor against the limit the executor knows for it, and
raises `IndexError` naming the op, the parameter, the first bad element and its value, before anything is launched.
Steps run eagerly while it is attached (no CUDA-graph replay) and every check synchronises, so this is a debugging aid,
not a serving mode. `FB_DEBUG_BOUNDS=1` attaches it to every engine built in the process.

    chk = BoundsChecker(engine)
    engine.forward(segments)
    chk.detach(); print(chk.checked)          # how many index tensors were looked at, per op

The role of the reference's bounds-checked debug kernels that write `ST_BOUNDS` (`crates/fe-cuda/src/lib.rs:299-343`),
moved in front of the launch: the check cannot fault, and it also covers the CPU ops.
"""
from __future__ import annotations

import inspect
from typing import Any, Callable, Dict, Optional, Tuple

import torch


def _limits(ex) -> Dict[str, Tuple[int, int, str]]:
    """Parameter name -> (lowest legal value, one past the highest, what the limit is)."""
    c, e = ex.cfg, ex.ecfg
    n_pages = next(iter(ex.k_cache.values())).shape[0] if ex.k_cache else 0
    lim = {
        "row_slot": (0, e.n_slots, "slots"), "seg_slot": (0, e.n_slots, "slots"),
        "row_pos": (0, e.max_ctx, "context positions"), "row_cpos": (0, e.max_ctx, "context positions"),
        "seg_pos0": (0, e.max_ctx, "context positions"), "row_kvlen": (0, e.max_ctx + 1, "context length"),
        "block_table": (-1, n_pages, "KV pages"),
    }
    return lim


# (op name, parameter) pairs whose limit depends on the op rather than on the parameter's name
def _special(ex, op: str, param: str, bound: Dict[str, Any]) -> Optional[Tuple[int, int, str]]:
    if op == "embed" and param == "ids":
        return 0, int(bound["table"].shape[0]), "rows of the embedding table"
    if op in ("moe_experts",) and param == "ids":
        return 0, max(1, ex.full_cfg.n_experts) + 1, "experts (+ the shared expert's stack entry)"
    if param == "row_parent":
        return -1, 1 << 30, "tree rows"
    return None


class _CheckedOps:
    def __init__(self, ops, ex, counts: Dict[str, int]):
        object.__setattr__(self, "_ops", ops)
        object.__setattr__(self, "_ex", ex)
        object.__setattr__(self, "_counts", counts)
        object.__setattr__(self, "_sigs", {})
        object.__setattr__(self, "_lim", _limits(ex))

    def __setattr__(self, name, value):
        setattr(self._ops, name, value)

    def __getattr__(self, name: str) -> Any:
        attr = getattr(self._ops, name)
        if not callable(attr) or name.startswith("_") or name in ("status",):
            return attr
        sig = self._sigs.get(name)
        if sig is None:
            try:
                sig = inspect.signature(attr)
            except (TypeError, ValueError):
                sig = False
            self._sigs[name] = sig
        if sig is False:
            return attr

        def checked(*a, **kw):
            try:
                bound = sig.bind(*a, **kw).arguments
            except TypeError:
                return attr(*a, **kw)                       # the call itself reports its argument error
            for param, val in bound.items():
                if not isinstance(val, torch.Tensor) or val.dtype not in (torch.int32, torch.int64) or val.numel() == 0:
                    continue
                lim = _special(self._ex, name, param, bound) or self._lim.get(param)
                if lim is None:
                    continue
                lo, hi, what = lim
                self._counts[name] = self._counts.get(name, 0) + 1
                bad = (val < lo) | (val >= hi)
                if bool(bad.any()):
                    flat = bad.reshape(-1).nonzero()[0].item()
                    idx = tuple(int(i) for i in torch.unravel_index(torch.tensor(flat), val.shape)) if val.dim() > 1 else (flat,)
                    raise IndexError(f"{name}: {param}{list(idx)} = {int(val.reshape(-1)[flat])} is outside [{lo}, {hi}) ({what})")
            return attr(*a, **kw)
        return checked


class BoundsChecker:
    def __init__(self, engine):
        self.ex = engine.ex
        self.checked: Dict[str, int] = {}
        self._orig = self.ex.ops
        self._orig_profile = self.ex.profile
        self.ex.ops = _CheckedOps(self._orig, self.ex, self.checked)
        if self.ex.profile is None:
            self.ex.profile = {}                            # a set profile makes the executor run eagerly

    def detach(self) -> None:
        self.ex.ops = self._orig
        self.ex.profile = self._orig_profile
