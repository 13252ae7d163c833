"""Pipeline schedules: which (stage, microbatch, fwd/bwd) task each pipeline rank runs, in order.

A schedule is pure Python and knows nothing about tensors.  ``schedule.tasks(n)`` returns one
list per pipeline rank; entries are :class:`Task`, :class:`FusedTask` (tasks that the runtime
launches as one unit, e.g. the last stage's forward and backward of the same microbatch) or
``None`` (an idle slot, which consumers strip).  The compiler list-schedules the unrolled
microbatch loop against these per-rank orders.

Behavioural parity with the reference's schedule module (src/jaxpp/schedules.py): the same
class names, constructor arguments, validation messages, stage→rank maps
(identity :204, round-robin :235, V-shape :636) and the same per-rank task orders for
``Std1F1B`` (:240), ``Eager1F1B`` (:277), ``GPipe`` (:316), ``ZeroBubble`` (:347),
``Interleaved1F1B`` (:451), ``KimiK2`` (:559) and ``DualPipeV`` (:623).  The orders here are
produced by per-rank generators written as phase lists (warm-up / steady / cool-down) rather
than by filling a time grid.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Iterable, Iterator, Sequence

from .types import MpmdIdx, TaskType

FWD = TaskType.FWD
BWD = TaskType.BWD
BWD_I = TaskType.BWD_I
BWD_W = TaskType.BWD_W


@dataclass(frozen=True)
class Task:
    stage_id: int
    mubatch_idx: int
    fwd_or_bwd: TaskType
    latency: int = field(hash=False, compare=False, default=0)

    @classmethod
    def make(cls, stage_id: int, mubatch_idx: int, fwd_or_bwd: TaskType, latency: int | None = None) -> "Task":
        return cls(stage_id, mubatch_idx, fwd_or_bwd, fwd_or_bwd.default_latency if latency is None else latency)

    def __str__(self) -> str:
        return mk_task_name(self.stage_id, self.fwd_or_bwd, self.mubatch_idx)


class FusedTask(tuple):
    """Several tasks that one rank runs back to back as a single launch unit."""

    @property
    def latency(self) -> int:
        return sum(t.latency for t in self)

    def __str__(self) -> str:
        return f"FusedTask({', '.join(str(t) for t in self)})"


ScheduleTasks = list  # list[list[Task | FusedTask | None]]

_PREFIX = {FWD: "fwd_", BWD: "bwd_", BWD_I: "bwdA_", BWD_W: "bwdW_"}


def mk_task_name(stage_id, ty: TaskType, mubatch_idx: int | None = None) -> str:
    """``fwd_3__5`` = forward of stage 3 on microbatch 5; ``bwdA_``/``bwdW_`` are the split halves."""
    tail = "" if mubatch_idx is None else f"__{mubatch_idx}"
    return f"{_PREFIX[ty]}{stage_id}{tail}"


class _Counter:
    """Hands out tasks with consecutive microbatch indices per (stage, kind)."""

    def __init__(self, split_bwd: bool = False):
        self.next_mb: dict[tuple[int, TaskType], int] = {}
        self.split_bwd = split_bwd

    def count(self, stage: int, kind: TaskType) -> int:
        return self.next_mb.get((stage, kind), 0)

    def take(self, stage: int, kind: TaskType) -> Task:
        mb = self.next_mb.get((stage, kind), 0)
        self.next_mb[(stage, kind)] = mb + 1
        return Task.make(stage, mb, kind)

    def fwd(self, stage: int) -> Task:
        return self.take(stage, FWD)

    def bwd_parts(self, stage: int) -> tuple[Task, ...]:
        """The whole backward of the next microbatch: one BWD task, or (BWD_I, BWD_W)."""
        if self.split_bwd:
            return (self.take(stage, BWD_I), self.take(stage, BWD_W))
        return (self.take(stage, BWD),)

    def bwd(self, stage: int):
        parts = self.bwd_parts(stage)
        return parts[0] if len(parts) == 1 else FusedTask(parts)

    def fwd_bwd(self, fwd_stage: int, bwd_stage: int) -> FusedTask:
        parts = self.bwd_parts(bwd_stage)
        return FusedTask((self.fwd(fwd_stage), *parts))


@dataclass(eq=True, frozen=True)
class BaseSchedule:
    num_stages: int
    is_partial_bwd: bool = field(default=False, init=False)

    def __post_init__(self):
        if self.num_stages <= 0:
            raise ValueError("The argument `num_stages` must be `>= 0`")

    # number of pipeline ranks the schedule produces lists for
    @property
    def num_ranks(self) -> int:
        return getattr(self, "mpmd_dim", self.num_stages)

    def get_mpmd_idx(self, stage_id: int) -> MpmdIdx:
        return MpmdIdx(stage_id)

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        raise NotImplementedError

    def ideal_bubble_fraction(self, n_mubatches: int) -> float:
        """Idle share of a rank's timeline with the integer latencies (FWD 1, BWD 2, halves 1).

        Found by replaying the per-rank orders under their data dependencies; used by the
        benchmark to compare a measured bubble with what the schedule allows.
        """
        return simulate_bubble(self, n_mubatches)


def _set(obj, name, value):
    object.__setattr__(obj, name, value)  # frozen dataclass


@dataclass(eq=True, frozen=True)
class InterleavedBaseSchedule(BaseSchedule):
    mpmd_dim: int = 0

    def __post_init__(self):
        super().__post_init__()
        if self.mpmd_dim <= 0:
            raise ValueError("The argument `mpmd_dim` must be `>= 0`")
        if self.num_stages % self.mpmd_dim != 0:
            raise ValueError(
                f"{self.num_stages=} can not be evenly divided by {self.mpmd_dim=}. "
                f"Remainder: {divmod(self.num_stages, self.mpmd_dim)=}"
            )

    def get_mpmd_idx(self, stage_id: int) -> MpmdIdx:
        return MpmdIdx(stage_id % self.mpmd_dim)


def _one_f_one_b(stage: int, n: int, warmup: int) -> list[Task]:
    """``warmup`` forwards, then backward/forward alternation, then the remaining backwards."""
    warmup = min(warmup, n)
    seq = [Task.make(stage, m, FWD) for m in range(warmup)]
    for k in range(n):
        seq.append(Task.make(stage, k, BWD))
        if warmup + k < n:
            seq.append(Task.make(stage, warmup + k, FWD))
    return seq


@dataclass(eq=True, frozen=True)
class Std1F1B(BaseSchedule):
    """PipeDream-flush 1F1B: rank ``r`` of ``S`` runs ``S - r`` warm-up forwards."""

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        S = self.num_stages
        return [_one_f_one_b(r, n_mubatches, S - r) for r in range(S)]


@dataclass(eq=True, frozen=True)
class Eager1F1B(BaseSchedule):
    """1F1B with ``2·(S-1-r)+1`` warm-up forwards, so that sends can run one step ahead."""

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        S = self.num_stages
        return [_one_f_one_b(r, n_mubatches, 2 * (S - 1 - r) + 1) for r in range(S)]


@dataclass(eq=True, frozen=True)
class GPipe(BaseSchedule):
    """All forwards, then all backwards."""

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        return [
            [Task.make(r, m, FWD) for m in range(n_mubatches)]
            + [Task.make(r, m, BWD) for m in range(n_mubatches)]
            for r in range(self.num_stages)
        ]


@dataclass(eq=True, frozen=True)
class ZeroBubble(BaseSchedule):
    """ZB-H1: backward split into an activation half (BWD_I) and a weight half (BWD_W);
    weight halves fill what would be bubbles in 1F1B."""

    def __post_init__(self):
        super().__post_init__()
        _set(self, "is_partial_bwd", True)

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        return self.build_schedule(n_mubatches)

    def build_schedule(self, n: int) -> ScheduleTasks:
        S = self.num_stages
        assert n >= S, (
            f"Expect num of microbatches >= num of stages, but {n} microbatches and {S} stages found"
        )
        return [self._rank(r, n) for r in range(S)]

    def _rank(self, r: int, n: int) -> list[Task]:
        S = self.num_stages
        c = _Counter()
        seq = [c.take(r, FWD) for _ in range(S - r)]
        # r rounds of (activation-backward, forward) while upstream ranks are still warming up
        for _ in range(r):
            seq.append(c.take(r, BWD_I))
            seq.append(c.take(r, FWD))
        # steady state and drain: rotate BWD_I → BWD_W → FWD, skipping kinds that are used up
        order = (BWD_I, BWD_W, FWD)
        pos = 0
        remaining = 3 * n - len(seq)
        while remaining:
            for probe in range(3):
                kind = order[(pos + probe) % 3]
                if c.count(r, kind) < n:
                    seq.append(c.take(r, kind))
                    pos = (pos + probe + 1) % 3
                    break
            else:  # pragma: no cover - remaining > 0 guarantees a kind is available
                raise ValueError("All tasks have been already scheduled for all mubatches")
            remaining -= 1
        return seq


@dataclass(eq=True, frozen=True)
class Interleaved1F1B(InterleavedBaseSchedule):
    """Megatron-style interleaved 1F1B: each rank owns ``num_stages / mpmd_dim`` virtual stages.

    The last stage's forward and backward of a microbatch are always one :class:`FusedTask`;
    with ``fuse_steady_state=True`` every steady-state (forward, backward) pair is fused.
    """

    fuse_steady_state: bool = False

    def __post_init__(self):
        super().__post_init__()
        _set(self, "vp", self.num_stages // self.mpmd_dim)
        _set(self, "is_partial_bwd", False)

    # -- phase sizes -------------------------------------------------------------------
    def microbatches_per_round(self, n_microbatches: int) -> int:
        rounds = max(1, n_microbatches // self.mpmd_dim)
        per_round, rem = divmod(n_microbatches, rounds)
        if rem != 0:
            raise ValueError("n_microbatches must be divisible by mpmd_dim")
        return per_round

    def _get_rank_warmup_ops(self, mpmd_idx: int, n_microbatches: int) -> int:
        per_round = self.microbatches_per_round(n_microbatches)
        # the last rank warms up (vp-1) rounds; every hop towards rank 0 adds two more forwards
        return (self.vp - 1) * per_round + 2 * (self.mpmd_dim - 1 - mpmd_idx)

    def get_rank_warmup_ops(self, mpmd_idx: int, n_microbatches: int) -> int:
        return min(self._get_rank_warmup_ops(mpmd_idx, n_microbatches), n_microbatches * self.vp)

    def _fwd_stage(self, rank: int, step: int, per_round: int) -> int:
        return ((step // per_round) % self.vp) * self.mpmd_dim + rank

    def _bwd_stage(self, rank: int, step: int, warmup: int, per_round: int) -> int:
        chunk = self.vp - 1 - ((step - warmup) // per_round) % self.vp
        return chunk * self.mpmd_dim + rank

    def _tasks_for_rank(self, rank: int, n: int) -> list:
        total = self.vp * n
        warmup = self.get_rank_warmup_ops(rank, n)
        per_round = self.microbatches_per_round(n)
        c = _Counter(split_bwd=self.is_partial_bwd)
        seq: list = []
        for step in range(total + warmup):
            has_fwd = step < total
            has_bwd = step >= warmup
            f = self._fwd_stage(rank, step, per_round) if has_fwd else None
            b = self._bwd_stage(rank, step, warmup, per_round) if has_bwd else None
            if has_fwd and has_bwd:
                if self.fuse_steady_state or f == self.num_stages - 1:
                    seq.append(c.fwd_bwd(f, b))
                else:
                    seq.append(c.fwd(f))
                    seq.append(c.bwd(b))
            elif has_fwd:
                seq.append(c.fwd(f))
            else:
                seq.append(c.bwd(b))
        return seq

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        return [self._tasks_for_rank(r, n_mubatches) for r in range(self.mpmd_dim)]


class KimiK2(Interleaved1F1B):
    """Interleaved 1F1B with one extra warm-up forward per rank."""

    def _get_rank_warmup_ops(self, mpmd_idx: int, n_microbatches: int) -> int:
        return super()._get_rank_warmup_ops(mpmd_idx, n_microbatches) + 1


@dataclass(eq=True, frozen=True)
class InterleavedGPipe(InterleavedBaseSchedule):
    """All forwards of every virtual stage (round-robin over chunks per group of ``mpmd_dim``
    microbatches), then all backwards in the mirrored order."""

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        P = self.mpmd_dim
        vp = self.num_stages // P
        out = []
        for r in range(P):
            fwd, bwd = [], []
            for start in range(0, n_mubatches, P):
                group = range(start, min(start + P, n_mubatches))
                for chunk in range(vp):
                    fwd.extend(Task.make(chunk * P + r, m, FWD) for m in group)
                for chunk in reversed(range(vp)):
                    bwd.extend(Task.make(chunk * P + r, m, BWD) for m in group)
            out.append(fwd + bwd)
        return out


def dualpipev_tasks(mpmd_dim: int, mpmd_idx: int, n_mubatches: int) -> list:
    """Task order of one rank under DualPipeV (the "cut-in-half" DualPipe of DeepSeek-V3).

    Rank ``r`` of ``P`` owns stage ``r`` (the descending arm of the V, called *near* below) and
    stage ``2P-1-r`` (the ascending arm, *far*).  The eight phases below follow the published
    DualPipeV algorithm; forward/backward pairs that overlap are emitted as fused tasks.
    """
    P, r, n = mpmd_dim, mpmd_idx, n_mubatches
    near, far = r, 2 * P - 1 - r
    c = _Counter(split_bwd=True)
    seq: list = []
    behind = P - 1 - r  # ranks between this one and the tip of the V

    # 1. forwards of the near stage only
    seq += [c.fwd(near) for _ in range(2 * behind)]
    # 2. alternate near / far forwards
    for _ in range(r + 1):
        seq += [c.fwd(near), c.fwd(far)]
    # 3. far backward (split, weight half right behind) followed by a far forward
    for _ in range(behind):
        seq += [c.take(far, BWD_I), c.take(far, BWD_W), c.fwd(far)]
    # 4. main loop: (near fwd ∥ far bwd) then (far fwd ∥ near bwd)
    for k in range(n - 2 * P + r + 1):
        if k == 0 and r == P - 1:
            seq += [c.fwd(near), c.bwd(far)]
        else:
            seq.append(c.fwd_bwd(near, far))
        seq.append(c.fwd_bwd(far, near))
    # 5. far backward, then (far fwd ∥ near bwd)
    for _ in range(behind):
        seq.append(c.bwd(far))
        seq.append(c.fwd_bwd(far, near))
    # 6. far / near backwards; the second half defers weight halves on alternating ranks
    rounds = r + 1
    zb_from = rounds // 2
    for k in range(rounds):
        defer = k >= zb_from
        seq.append(c.take(far, BWD_I) if defer and r % 2 == 1 else c.bwd(far))
        # the first stage's backward is never split (nothing upstream needs its input grads)
        seq.append(c.take(near, BWD_I) if defer and r % 2 == 0 and near != 0 else c.bwd(near))
    # 7. near activation backwards
    for _ in range(behind):
        seq.append(c.bwd(near) if near == 0 else c.take(near, BWD_I))
    # 8. all weight halves still owed, oldest microbatch first
    owed = []
    for stage in sorted({near, far}):
        owed += [(m, stage) for m in range(c.count(stage, BWD_W), n)]
    # consume in (microbatch, stage) order
    for m, stage in sorted(owed):
        t = c.take(stage, BWD_W)
        assert t.mubatch_idx == m
        seq.append(t)
    return seq


@dataclass(eq=True, frozen=True)
class DualPipeV(InterleavedBaseSchedule):
    def __post_init__(self):
        super().__post_init__()
        if self.num_stages != 2 * self.mpmd_dim:
            raise ValueError(
                f"{DualPipeV.__name__} only supports 2 * mpmd_dim stages,"
                f" {self.num_stages=} requested with {self.mpmd_dim=}"
            )
        _set(self, "is_partial_bwd", True)

    def get_mpmd_idx(self, stage_id: int) -> MpmdIdx:
        arm, pos = divmod(stage_id, self.mpmd_dim)
        return MpmdIdx(pos if arm % 2 == 0 else self.mpmd_dim - 1 - pos)

    def tasks(self, n_mubatches: int) -> ScheduleTasks:
        if not (n_mubatches > 0 and n_mubatches >= self.num_stages):
            raise ValueError(
                f"{DualPipeV.__name__} requires {n_mubatches=} >= "
                f"{self.num_stages=} ({self.mpmd_dim=})"
            )
        return [dualpipev_tasks(self.mpmd_dim, r, n_mubatches) for r in range(self.mpmd_dim)]


# ---------------------------------------------------------------------------------------
# Normalisation used by the compiler (reference: schedules.py:660-739)
# ---------------------------------------------------------------------------------------

def strip_nones(ts: Iterable) -> list:
    return [t for t in ts if t is not None]


def unpack_fused_tasks_fn(ts: Iterable) -> list:
    flat = []
    for t in ts:
        flat.extend(t) if isinstance(t, FusedTask) else flat.append(t)
    return flat


def merge_first_stage_bwd(tasks: Sequence, first_stage_id: Any) -> list:
    """Merge ``BWD_I`` + ``BWD_W`` of the first stage into one task typed ``BWD_I``.

    The first stage has no upstream consumer of input gradients, so its backward cannot be
    split by dataflow; every schedule must therefore emit the two halves adjacent
    (``NotImplementedError`` otherwise).  The merged task carries the summed latency.
    """
    out: list = []
    i = 0
    tasks = list(tasks)
    while i < len(tasks):
        t = tasks[i]
        if isinstance(t, FusedTask):
            inner = merge_first_stage_bwd(list(t), first_stage_id)
            out.append(inner[0] if len(inner) == 1 else FusedTask(inner))
            i += 1
            continue
        if t.stage_id == first_stage_id and t.fwd_or_bwd is BWD_I:
            nxt = tasks[i + 1] if i + 1 < len(tasks) else None
            ok = (
                nxt is not None
                and not isinstance(nxt, FusedTask)
                and nxt.stage_id == first_stage_id
                and nxt.fwd_or_bwd is BWD_W
            )
            if not ok:
                raise NotImplementedError(
                    f"{BWD_I} is not followed by {BWD_W} for first_stage {first_stage_id} "
                    f"at tasks {i} {[str(x) for x in tasks[i:i + 2]]}.\n{[str(x) for x in tasks]}"
                )
            out.append(dataclasses.replace(t, latency=t.latency + nxt.latency))
            i += 2
            continue
        out.append(t)
        i += 1
    return out


# name kept for API parity with the reference
check_and_strip_adjecent_bwd_a_bwd_w = merge_first_stage_bwd


def preprocess_schedule_tasks(schedule: ScheduleTasks, first_stage_id, unpack_fused_tasks: bool) -> list[list]:
    per_rank = [strip_nones(ts) for ts in schedule]
    if unpack_fused_tasks:
        per_rank = [unpack_fused_tasks_fn(ts) for ts in per_rank]
    return [merge_first_stage_bwd(ts, first_stage_id) for ts in per_rank]


# ---------------------------------------------------------------------------------------
# Dependency replay: validity check and ideal bubble
# ---------------------------------------------------------------------------------------

def _deps(t: Task, num_stages: int, partial: bool, merged_first: bool) -> list[tuple[int, int, TaskType]]:
    """Tasks that must finish before ``t`` starts (keys: stage, microbatch, kind)."""
    s, m, k = t.stage_id, t.mubatch_idx, t.fwd_or_bwd
    bwd_in = BWD_I if partial else BWD
    if k is FWD:
        return [(s - 1, m, FWD)] if s > 0 else []
    if k is BWD_W:
        return [(s, m, BWD_I)]
    deps = [(s, m, FWD)]
    if s < num_stages - 1:
        deps.append((s + 1, m, bwd_in))
    return deps


def replay(schedule: BaseSchedule, n_mubatches: int, unpack_fused: bool = False):
    """List-schedule the per-rank orders under data dependencies with integer latencies.

    Returns ``(makespan, busy_per_rank, timeline)`` where ``timeline[rank]`` is a list of
    ``(start, end, task_or_fused)``.  Raises ``AssertionError`` if the orders deadlock.
    """
    per_rank = preprocess_schedule_tasks(schedule.tasks(n_mubatches), 0, unpack_fused)
    S = schedule.num_stages
    partial = schedule.is_partial_bwd
    done: dict[tuple[int, int, TaskType], int] = {}
    cursor = [0] * len(per_rank)
    clock = [0] * len(per_rank)
    timeline: list[list] = [[] for _ in per_rank]
    total = sum(len(ts) for ts in per_rank)
    placed = 0
    while placed < total:
        best = None
        for r, ts in enumerate(per_rank):
            if cursor[r] >= len(ts):
                continue
            unit = ts[cursor[r]]
            members = list(unit) if isinstance(unit, FusedTask) else [unit]
            inside = set()
            ready = clock[r]
            ok = True
            for t in members:
                for d in _deps(t, S, partial, True):
                    if d in inside:
                        continue
                    if d not in done:
                        ok = False
                        break
                    ready = max(ready, done[d])
                if not ok:
                    break
                inside.add((t.stage_id, t.mubatch_idx, t.fwd_or_bwd))
            if ok and (best is None or ready < best[0]):
                best = (ready, r, unit, members)
        if best is None:
            raise AssertionError("Schedule does not honor data dependencies")
        start, r, unit, members = best
        end = start + sum(t.latency for t in members)
        for t in members:
            done[(t.stage_id, t.mubatch_idx, t.fwd_or_bwd)] = end
            if t.fwd_or_bwd is BWD_I and t.latency > 1:  # merged first-stage backward
                done[(t.stage_id, t.mubatch_idx, BWD_W)] = end
        clock[r] = end
        cursor[r] += 1
        placed += 1
        timeline[r].append((start, end, unit))
    makespan = max(clock)
    busy = [sum(e - s for s, e, _ in tl) for tl in timeline]
    return makespan, busy, timeline


def simulate_bubble(schedule: BaseSchedule, n_mubatches: int) -> float:
    makespan, busy, _ = replay(schedule, n_mubatches)
    return 1.0 - (sum(busy) / len(busy)) / makespan


__all__ = [
    "Task", "FusedTask", "BaseSchedule", "InterleavedBaseSchedule", "Std1F1B", "Eager1F1B", "GPipe",
    "ZeroBubble", "Interleaved1F1B", "KimiK2", "InterleavedGPipe", "DualPipeV", "dualpipev_tasks",
    "preprocess_schedule_tasks", "mk_task_name", "replay", "simulate_bubble",
]
