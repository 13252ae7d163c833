"""Per-rank task timeline of one pipelined step, from the CUDA events the executor records around every task.

The reference wraps each task in a profiler annotation and leaves the timeline to an external trace viewer
(src/jaxpp/jax_primitives.py:844-846); here the events are read back after the step and summarised as text:
per task kind (``fwd_3``, ``bwd_3``, ``bwdA_3``, fused groups, ``before_loop``, ``after_loop``) the number of
instances, their mean and total duration, and the idle time of the compute stream in front of them — which, on a
pipeline rank, is time spent waiting for an activation or a gradient from another rank.
"""
from __future__ import annotations

import re
from collections import OrderedDict

_MB = re.compile(r"__\d+")


def task_kind(name: str) -> str:
    """``fwd_3__17`` -> ``fwd_3``; ``fused_fwd_7__2_bwd_7__2`` -> ``fused_fwd_7_bwd_7``; ``after_loop_r2_0`` stays."""
    return _MB.sub("", name)


def summarise_events(events, step_start=None, step_end=None) -> dict:
    """``events`` is ``RankState.events`` (``(task name, start event, end event)`` in launch order) of a step that was
    run with ``record_events=True`` and has been synchronised.  Returns ``{"kinds": {kind: {...}}, "busy_ms", "idle_ms",
    "step_ms"}``; ``step_start`` / ``step_end`` are CUDA events recorded around the step on the same stream."""
    kinds: "OrderedDict[str, dict]" = OrderedDict()
    prev_end = step_start
    busy = idle = 0.0
    for name, e0, e1 in events:
        ms = e0.elapsed_time(e1)
        gap = prev_end.elapsed_time(e0) if prev_end is not None else 0.0
        gap = max(0.0, gap)
        k = kinds.setdefault(task_kind(name), {"n": 0, "total_ms": 0.0, "wait_before_ms": 0.0, "max_ms": 0.0})
        k["n"] += 1
        k["total_ms"] += ms
        k["wait_before_ms"] += gap
        k["max_ms"] = max(k["max_ms"], ms)
        busy += ms
        idle += gap
        prev_end = e1
    tail = max(0.0, prev_end.elapsed_time(step_end)) if (step_end is not None and prev_end is not None) else 0.0
    step_ms = step_start.elapsed_time(step_end) if (step_start is not None and step_end is not None) else busy + idle
    for k in kinds.values():
        k["mean_ms"] = k["total_ms"] / max(1, k["n"])
    return {"kinds": kinds, "busy_ms": busy, "idle_ms": idle + tail, "tail_ms": tail, "step_ms": step_ms}


def format_summary(rank_label: str, summary: dict) -> str:
    lines = [f"{rank_label}: step {summary['step_ms']:.1f} ms, tasks {summary['busy_ms']:.1f} ms, "
             f"idle {summary['idle_ms']:.1f} ms ({100 * summary['idle_ms'] / max(summary['step_ms'], 1e-9):.1f} %)",
             f"  {'task kind':<34}{'n':>5}{'mean ms':>10}{'max ms':>10}{'total ms':>11}{'% step':>8}{'idle before ms':>16}"]
    for kind, k in summary["kinds"].items():
        lines.append(f"  {kind:<34}{k['n']:>5}{k['mean_ms']:>10.3f}{k['max_ms']:>10.3f}{k['total_ms']:>11.1f}"
                     f"{100 * k['total_ms'] / max(summary['step_ms'], 1e-9):>8.1f}{k['wait_before_ms']:>16.1f}")
    return "\n".join(lines)
