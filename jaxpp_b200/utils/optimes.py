"""Per-op device time inside the tasks of a step, from CUDA events recorded around every op call.

``collect_task_times_ms`` costs whole tasks; this costs the ops inside them, under the conditions of a real step
(warm caches, the power cap, the clocks of a long run), which a kernel profiler that serialises and replays launches
does not reproduce.  While ``collecting()`` is active, task code is bound with every call target wrapped: the wrapper
records an event before and after the call on the current stream; ``table()`` reads them back after a synchronise.
An op that launches several kernels (a norm backward and its partial-sum reduction, say) is one row.  Event records
cost a few microseconds of stream time each, so the step itself runs slightly longer than an uninstrumented one:
read the shares, not the absolute step time.
"""
from __future__ import annotations

import contextlib
from collections import OrderedDict

import torch

ACTIVE = [False]
_RECORDS: list = []     # (op name, start event, end event)


def name_of(target) -> str:
    n = str(target)
    for prefix in ("b200.", "b200tp.", "b200dp.", "b200moe.", "b200cp.", "aten."):
        if n.startswith(prefix):
            return n[:-len(".default")] if n.endswith(".default") else n
    return getattr(target, "__name__", n)


class Timed:
    """Callable stand-in for an op overload that brackets every call with CUDA events."""

    def __init__(self, target, name: str | None = None):
        self.target = target
        self.name = name or name_of(target)

    def __call__(self, *args, **kwargs):
        if not ACTIVE[0] or not torch.cuda.is_available():
            return self.target(*args, **kwargs)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = self.target(*args, **kwargs)
        e1.record()
        _RECORDS.append((self.name, e0, e1))
        return out


def unwrap(target):
    return target.target if isinstance(target, Timed) else target


@contextlib.contextmanager
def collecting():
    prev = ACTIVE[0]
    ACTIVE[0] = True
    _RECORDS.clear()
    try:
        yield
    finally:
        ACTIVE[0] = prev


def table(synchronize: bool = True) -> "OrderedDict[str, dict]":
    """``{op: {"n", "total_ms", "mean_us"}}`` of the calls recorded since ``collecting()`` was entered, largest first."""
    if synchronize and torch.cuda.is_available():
        torch.cuda.synchronize()
    agg: dict = {}
    for name, e0, e1 in _RECORDS:
        row = agg.setdefault(name, {"n": 0, "total_ms": 0.0})
        row["n"] += 1
        row["total_ms"] += e0.elapsed_time(e1)
    for row in agg.values():
        row["mean_us"] = 1e3 * row["total_ms"] / max(1, row["n"])
    return OrderedDict(sorted(agg.items(), key=lambda kv: -kv[1]["total_ms"]))


def format_table(rows, step_ms: float, title: str = "") -> str:
    covered = sum(r["total_ms"] for r in rows.values())
    lines = [title] if title else []
    lines.append(f"{'op':<34}{'calls':>8}{'mean us':>11}{'total ms':>11}{'% of step':>11}")
    for name, r in rows.items():
        lines.append(f"{name:<34}{r['n']:>8}{r['mean_us']:>11.1f}{r['total_ms']:>11.2f}{100 * r['total_ms'] / step_ms:>11.2f}")
    lines.append(f"{'(between ops: launch gaps, waits)':<34}{'':>8}{'':>11}{step_ms - covered:>11.2f}{100 * (step_ms - covered) / step_ms:>11.2f}")
    lines.append(f"{'step':<34}{'':>8}{'':>11}{step_ms:>11.2f}{100.0:>11.2f}")
    return "\n".join(lines)
