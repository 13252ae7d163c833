"""Interpreters for compiled programs.

``RankState`` holds one pipeline rank's value environment and executes that rank's instructions;
``run_single_controller`` drives all ranks of a program from one process in the program's global
order (the oracle / CPU simulator, and the mode notebooks use; reference:
``GlobalMpmdFunction.__call__``, src/jaxpp/core.py:3709-3793); ``run_multi_controller`` executes
only this process's rank and talks to the others through a :class:`~.comm.Comm` (reference:
``ScalarMpmdFunction.__call__``, :3401-3447, and the eager primitive implementations in
src/jaxpp/jax_primitives.py:370-523, 776-859).
"""
from __future__ import annotations

import contextlib
import os
import time
from collections import defaultdict
from typing import Any, Sequence

import torch

from ..compiler.program import (Accum, AllGather, AllReduce, Delete, LoopIndex, Program, RunTask, SendDone,
                                Slice, Transfer)
from .. import fault
from ..utils import config

# ---- task timing (reference: collect_task_times_ms, jax_primitives.py:742-773) -----------------
_TIMES: list[dict] = []


@contextlib.contextmanager
def collect_task_times_ms(enabled: bool = True):
    """Collect ``task name → [milliseconds…]`` for every task run inside the ``with``.

    While active, the executor synchronises the device before and after each task, which serialises
    the pipeline: use it to cost tasks, not to measure throughput.
    """
    if not enabled:
        yield None
        return
    table: dict[str, list[float]] = defaultdict(list)
    _TIMES.append(table)
    try:
        yield table
    finally:
        _TIMES.pop()


_SIDE_STREAMS: dict = {}
OVERLAPPED = [False]


def _side_stream(device: torch.device):
    s = _SIDE_STREAMS.get(device)
    if s is None:
        s = _SIDE_STREAMS[device] = torch.cuda.Stream(device)
    return s


@contextlib.contextmanager
def overlapped_collectives():
    """Inside: peer-memory collectives use their side-stream workspace (its flags and epochs are independent of the
    compute stream's, whose calls are ordered separately) and a small grid that shares the SMs with compute kernels."""
    prev = OVERLAPPED[0]
    OVERLAPPED[0] = True
    try:
        yield
    finally:
        OVERLAPPED[0] = prev


class RankState:
    """Environment and instruction semantics of one pipeline rank."""

    def __init__(self, rank: int, device: torch.device, record_events: bool = False):
        self.rank = rank
        self.device = device
        self.env: dict[int, torch.Tensor] = {}
        self.index_cache: dict[int, torch.Tensor] = {}
        self.record_events = record_events and device.type == "cuda"
        self.events: list[tuple[str, Any, Any]] = []
        self.pending_events: dict[int, Any] = {}   # value id -> CUDA event of the side-stream work that produces it

    # -- individual instructions --------------------------------------------------------------
    def run_task(self, ins: RunTask):
        env = self.env
        args = []
        for v, donate in zip(ins.ins, ins.donate):
            args.append(env.pop(v) if donate else env[v])
        if self.pending_events:
            for v in ins.ins:
                ev = self.pending_events.pop(v, None)
                if ev is not None:
                    torch.cuda.current_stream(self.device).wait_event(ev)
        fn = ins.code.bind(self.device)
        sink = None
        if ins.sinks:
            sink = {j: env[acc] for j, acc in ins.sinks if acc in env}
            for hook in ins.hooks:
                if hook[0] in sink:
                    sink[hook[0]] = (sink[hook[0]], self._early_collective(hook))
        timing = _TIMES[-1] if _TIMES else None
        if timing is not None:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            t0 = time.perf_counter()
        if self.record_events:
            e0 = torch.cuda.Event(enable_timing=True)
            e0.record()
        if self.device.type == "cuda" and config.nvtx_ranges.value:
            torch.cuda.nvtx.range_push(ins.name)
            try:
                outs = fn(args, sink) if sink else fn(args)
            finally:
                torch.cuda.nvtx.range_pop()
        else:
            outs = fn(args, sink) if sink else fn(args)
        if self.record_events:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.events.append((ins.name, e0, e1))
        if timing is not None:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            timing[f"{ins.name} ({id(ins.code)})"].append((time.perf_counter() - t0) * 1e3)
        for v, o in zip(ins.outs, outs):
            if v >= 0:
                env[v] = o

    def _early_collective(self, hook):
        """The callable a weight-gradient sink runs once the last contribution is in the accumulator: launch the
        gradient collective on the side stream (ordered after the GEMM that was just enqueued) and leave its result
        in the environment for the after-loop task, which waits for the side stream's event."""
        _, _, result_vid, op, args = hook

        def run(acc: torch.Tensor):
            if self.device.type != "cuda":
                self.env[result_vid] = op(acc, *args)
                return
            main = torch.cuda.current_stream(self.device)
            side = _side_stream(self.device)
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(side):
                side.wait_event(ready)
                with overlapped_collectives():
                    out = op(acc, *args)
                done = torch.cuda.Event()
                done.record(side)
            acc.record_stream(side)     # read by the side stream after this task has dropped it
            out.record_stream(main)     # allocated on the side stream, consumed on the compute stream
            self.env[result_vid] = out
            self.pending_events[result_vid] = done

        return run

    def slice(self, ins: Slice):
        self.env[ins.out] = self.env[ins.src].select(ins.axis, ins.index)

    def loop_index(self, ins: LoopIndex):
        t = self.index_cache.get(ins.index)
        if t is None:
            t = torch.tensor(ins.index, dtype=torch.int64, device=self.device)
            self.index_cache[ins.index] = t
        self.env[ins.out] = t

    def accum(self, ins: Accum):
        env = self.env
        val = env[ins.val]
        acc = env.get(ins.acc)
        if ins.kind == 1:  # concat: write slot
            if acc is None:
                shape = list(val.shape)
                shape.insert(ins.axis, ins.n)
                acc = torch.empty(shape, dtype=val.dtype, device=val.device)
                env[ins.acc] = acc
            acc.select(ins.axis, ins.index).copy_(val)
            return
        if acc is None:
            env[ins.acc] = val if (ins.steal and val.is_contiguous()) else val.clone()
        elif acc is val:
            pass  # the task already added this microbatch's contribution into the accumulator (a sink)
        elif ins.kind == 0:
            acc.add_(val)
        else:
            torch.maximum(acc, val, out=acc)

    def delete(self, ins: Delete):
        for v in ins.vids:
            self.env.pop(v, None)

    def busy_ms(self) -> float:
        """Sum of task durations recorded with CUDA events (call after a device synchronise)."""
        return sum(e0.elapsed_time(e1) for _, e0, e1 in self.events)


def _local_sum(state: RankState, ins: AllReduce, like_shape, like_dtype):
    if ins.local:
        buf = state.env[ins.local[0]].clone()
        for v in ins.local[1:]:
            buf.add_(state.env[v])
        return buf
    return torch.zeros(like_shape, dtype=like_dtype, device=state.device)


LIVE_REPORT: list = []   # filled when JAXPP_B200_TRACK_LIVE_BYTES=1: one dict per step of this process


def _live_bytes(env: dict):
    """Bytes of distinct storages referenced by the environment, and the values sorted by size."""
    seen: dict[int, int] = {}
    items = []
    for vid, t in env.items():
        if not isinstance(t, torch.Tensor):
            continue
        st = t.untyped_storage()
        key = st.data_ptr()
        if key not in seen:
            seen[key] = st.nbytes()
            items.append((st.nbytes(), vid, tuple(t.shape), str(t.dtype)))
    return sum(seen.values()), sorted(items, reverse=True)


def run_single_controller(prog: Program, inputs: Sequence[torch.Tensor | None], devices: Sequence[torch.device],
                          record_events: bool = False) -> tuple[list[RankState], list]:
    """Execute ``prog`` for all ranks in this process.  ``inputs[i]`` is the full flat input ``i`` (or
    ``None`` if unused); returns the rank states and the flat outputs as ``{rank: tensor}`` dicts."""
    states = [RankState(r, devices[r], record_events) for r in range(prog.n_ranks)]
    for (vid, ranks), x in zip(prog.inputs, inputs):
        for r in ranks:
            states[r].env[vid] = x if x.device == devices[r] else x.to(devices[r])
    pending_collectives: dict[int, list] = defaultdict(list)
    track = os.environ.get("JAXPP_B200_TRACK_LIVE_BYTES") == "1"
    peak = {"bytes": 0}
    for pos, ins in enumerate(prog.instrs):
        st = states[ins.rank]
        if track and ins.rank == 0 and isinstance(ins, (RunTask, Delete)):
            total, items = _live_bytes(st.env)
            if total > peak["bytes"]:
                peak = {"bytes": total, "before": f"{pos}: {getattr(ins, 'name', type(ins).__name__)}", "largest": items[:12],
                        "all": items, "n_values": len(items), "rank": 0}
        if isinstance(ins, RunTask):
            st.run_task(ins)
        elif isinstance(ins, Slice):
            st.slice(ins)
        elif isinstance(ins, LoopIndex):
            st.loop_index(ins)
        elif isinstance(ins, Accum):
            st.accum(ins)
        elif isinstance(ins, Transfer):
            dst = states[ins.dst]
            for v in ins.vids:
                t = st.env[v]
                dst.env[v] = t if t.device == dst.device else t.to(dst.device, non_blocking=True)
        elif isinstance(ins, SendDone):
            pass
        elif isinstance(ins, Delete):
            st.delete(ins)
        elif isinstance(ins, (AllReduce, AllGather)):
            # a rank's contribution is read when *its* instruction is reached (it may be deleted right after)
            group = pending_collectives[ins.cid]
            if isinstance(ins, AllReduce):
                info = prog.values[ins.out]
                group.append((ins, _local_sum(st, ins, info.shape, info.dtype)))
            else:
                group.append((ins, {p: st.env[v] for p, v in ins.local.items()}))
            if len(group) == len(ins.ranks):
                _collective_single(states, group)
                del pending_collectives[ins.cid]
        else:  # pragma: no cover
            raise NotImplementedError(type(ins))
    if track:
        LIVE_REPORT.append(peak)
    outs = []
    for o in prog.outputs:
        if o[0] == "c":
            outs.append(o[1])
        else:
            _, vid, ranks = o
            outs.append({r: states[r].env[vid] for r in ranks})
    return states, outs


def _collective_single(states, group):
    first = group[0][0]
    if isinstance(first, AllReduce):
        home = states[first.ranks[0]].device
        total = None
        for ins, part in sorted(group, key=lambda g: g[0].rank):
            part = part.to(home)
            total = part if total is None else total.add_(part)
        for ins, _ in group:
            states[ins.rank].env[ins.out] = total.to(states[ins.rank].device).clone() if len(group) > 1 else total
    else:
        parts: dict[int, torch.Tensor] = {}
        for ins, local in group:
            parts.update(local)
        for ins, _ in group:
            dev = states[ins.rank].device
            states[ins.rank].env[ins.out] = torch.cat([parts[p].to(dev) for p in sorted(parts)], dim=ins.axis)


def run_multi_controller(prog: Program, rank: int, inputs: Sequence[torch.Tensor | None], device: torch.device, comm,
                         record_events: bool = False) -> tuple[RankState, list]:
    """Execute this process's part of ``prog``.  ``inputs[i]`` is the local tensor of flat input ``i`` or
    ``None`` when this rank does not hold it."""
    st = RankState(rank, device, record_events)
    for (vid, ranks), x in zip(prog.inputs, inputs):
        if rank in ranks:
            if x is None:
                raise ValueError(f"input %{vid} is required on pipeline rank {rank} but no local data was given")
            st.env[vid] = x
    comm.begin_step(st)
    track = os.environ.get("JAXPP_B200_TRACK_LIVE_BYTES") == "1"
    peak = {"bytes": 0}
    for pos, ins in enumerate(prog.for_rank(rank)):
        if track and isinstance(ins, (RunTask, Delete)):
            total, items = _live_bytes(st.env)
            if total > peak["bytes"]:
                grew = total > 1.05 * peak["bytes"]
                peak = {"bytes": total, "before": f"{pos}: {getattr(ins, 'name', type(ins).__name__)}", "largest": items[:12], "all": items,
                        "n_values": len(items)}
                if grew and device.type == "cuda" and total > 1e9:   # as it happens: a step that runs out of memory never reports
                    import sys
                    print(f"[live rank {rank}] env {total / 1e9:.1f} GB in {len(items)} values before {peak['before']}; allocator "
                          f"{torch.cuda.memory_allocated(device) / 1e9:.1f} GB now, {torch.cuda.max_memory_allocated(device) / 1e9:.1f} GB max; "
                          + "; ".join(f"%{v} {sh} {dt} {b / 1e9:.2f}GB" for b, v, sh, dt in items[:8]), file=sys.stderr, flush=True)
        if isinstance(ins, RunTask):
            if fault._PLAN[0] is not None:
                fault.maybe_fail_task(rank, ins.name)
            comm.before_use(st, ins.ins)
            st.run_task(ins)
        elif isinstance(ins, Slice):
            st.slice(ins)
        elif isinstance(ins, LoopIndex):
            st.loop_index(ins)
        elif isinstance(ins, Accum):
            comm.before_use(st, (ins.val,))
            st.accum(ins)
        elif isinstance(ins, Transfer):
            if ins.rank == rank:
                comm.send(st, ins, prog)
            else:
                comm.recv(st, ins, prog)
        elif isinstance(ins, SendDone):
            comm.send_done(st, ins)
        elif isinstance(ins, Delete):
            st.delete(ins)
        elif isinstance(ins, AllReduce):
            comm.before_use(st, ins.local)
            info = prog.values[ins.out]
            buf = _local_sum(st, ins, info.shape, info.dtype)
            st.env[ins.out] = comm.all_reduce(buf, ins.ranks)
        elif isinstance(ins, AllGather):
            comm.before_use(st, ins.local.values())
            st.env[ins.out] = comm.all_gather(st, ins, prog)
        else:  # pragma: no cover
            raise NotImplementedError(type(ins))
    comm.end_step(st)
    if track:
        peak["rank"] = rank
        LIVE_REPORT.append(peak)
    outs = []
    for o in prog.outputs:
        if o[0] == "c":
            outs.append(o[1])
        else:
            _, vid, ranks = o
            if rank in ranks:
                comm.before_use(st, (vid,))
            outs.append({rank: st.env[vid]} if rank in ranks else {})
    return st, outs
