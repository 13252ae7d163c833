"""The per-rank instruction set and the compiled program container.

A compiled train step is a *global* list of instructions, each tagged with the pipeline rank that
executes it, in a deadlock-free total order; the program of one rank is the sub-list with its
tag, with every ``Transfer`` seen as a send on its source rank and a receive on its target rank.
This is the counterpart of the reference's instruction set (src/jaxpp/jax_primitives.py: task,
transfer/send/recv, send_done, delete, all_reduce, all_gather) and of its per-rank program
extraction (src/jaxpp/core.py:2728-2896).  Values are named by integer ids; each rank keeps its
own id → tensor environment.
"""
from __future__ import annotations

import dataclasses
from typing import Any

import torch

from ..types import TaskType


@dataclasses.dataclass
class ValueInfo:
    vid: int
    shape: tuple[int, ...]
    dtype: torch.dtype
    label: str = ""

    @property
    def nbytes(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n * self.dtype.itemsize


@dataclasses.dataclass
class Instr:
    rank: int


@dataclasses.dataclass
class RunTask(Instr):
    """Run executable ``code`` on ``ins`` producing ``outs``; ``donate[i]`` ⇒ drop input i from the
    environment before the call (it is not used afterwards on this rank)."""

    name: str
    code: Any  # codegen.TaskCode
    ins: list[int]
    outs: list[int]
    donate: list[bool]
    stage_id: int | None = None
    task_type: TaskType | None = None
    mubatch: int | None = None
    start: int = 0  # list-scheduling clock (integer latencies)
    end: int = 0
    # (output position, accumulator value id): outputs that only feed the loop's Add accumulation and that the
    # task can add into the accumulator itself (weight gradients, see ops/sink.py)
    sinks: list = dataclasses.field(default_factory=list)
    # (output position, accumulator value id, result value id, collective op, its other arguments): a gradient
    # collective that the step applies to a loop accumulator after the loop, issued instead from inside this task --
    # the one that adds the last microbatch's contribution -- as soon as the weight-gradient GEMM has run, on a side
    # stream, so that it overlaps the rest of the backward pass (see lower.Lowering.plan_early_collectives)
    hooks: list = dataclasses.field(default_factory=list)


@dataclasses.dataclass
class Slice(Instr):
    """``out = env[src].select(axis, index)`` — microbatch ``index`` of a batched input (a view)."""

    out: int
    src: int
    axis: int
    index: int


@dataclasses.dataclass
class LoopIndex(Instr):
    """``out`` = 0-d int64 tensor holding the microbatch index."""

    out: int
    index: int


@dataclasses.dataclass
class Accum(Instr):
    """treduce accumulation of microbatch ``index``: kind 0 add, 1 concat (write slot), 2 max."""

    acc: int
    val: int
    kind: int
    axis: int
    index: int
    n: int
    steal: bool  # first microbatch may adopt ``val``'s buffer instead of copying


@dataclasses.dataclass
class Transfer(Instr):
    """Move ``vids`` from ``rank`` (source) to ``dst``.  ``tid`` increases monotonically in the
    global order and is identical on every process."""

    dst: int
    vids: list[int]
    tid: int


@dataclasses.dataclass
class SendDone(Instr):
    """All sends of transfer ``tid`` have completed; the source may reuse those buffers."""

    tid: int


@dataclasses.dataclass
class Delete(Instr):
    vids: list[int]


@dataclasses.dataclass
class AllReduce(Instr):
    """Cross-rank sum: every rank in ``ranks`` adds up its ``local`` operands (zeros if none) and the
    partial sums are all-reduced; ``out`` lives on all of ``ranks``.  One instruction per participant."""

    ranks: list[int]
    local: list[int]
    out: int
    cid: int


@dataclasses.dataclass
class AllGather(Instr):
    """Cross-rank concatenation along ``axis`` of ``n_parts`` operands; ``local`` maps operand position →
    vid for the operands this rank owns; ``owners[p]`` is the rank that contributes operand ``p``."""

    ranks: list[int]
    local: dict[int, int]
    owners: list[int]
    axis: int
    out: int
    cid: int


@dataclasses.dataclass
class Program:
    n_ranks: int
    instrs: list[Instr]
    values: dict[int, ValueInfo]
    # flat tensor input position → (vid, ranks that must hold it; empty = unused)
    inputs: list[tuple[int, tuple[int, ...]]]
    # flat output position → ("v", vid, ranks) | ("c", python constant)
    outputs: list[tuple]
    meta: dict = dataclasses.field(default_factory=dict)

    def for_rank(self, rank: int) -> list[Instr]:
        """Instructions that ``rank`` executes (transfers appear on both their endpoints)."""
        return [i for i in self.instrs if i.rank == rank or (isinstance(i, Transfer) and i.dst == rank)]

    # ---- text dump (reference: JAXPP_DUMP_DIR, core.py:3471-3484) ---------------------------
    def dump(self, rank: int | None = None) -> str:
        lines = []
        seq = self.instrs if rank is None else self.for_rank(rank)
        for ins in seq:
            lines.append(format_instr(ins, self.values, rank))
        return "\n".join(lines)

    def stats(self) -> dict:
        sent = sum(self.values[v].nbytes for i in self.instrs if isinstance(i, Transfer) for v in i.vids)
        return {
            "n_instrs": len(self.instrs),
            "n_tasks": sum(isinstance(i, RunTask) for i in self.instrs),
            "n_transfers": sum(isinstance(i, Transfer) for i in self.instrs),
            "transfer_bytes": sent,
            "n_executables": len({id(i.code) for i in self.instrs if isinstance(i, RunTask)}),
        }


def _v(values, vid):
    info = values.get(vid)
    if info is None:
        return f"%{vid}"
    dt = str(info.dtype).replace("torch.", "")
    return f"%{vid}:{dt}{list(info.shape)}"


def format_instr(ins: Instr, values, view_rank: int | None = None) -> str:
    r = f"[r{ins.rank}] "
    if isinstance(ins, RunTask):
        outs = ", ".join(_v(values, v) for v in ins.outs)
        inn = ", ".join(("~" if d else "") + f"%{v}" for v, d in zip(ins.ins, ins.donate))
        early = "".join(f" ; %{h[2]} = early {str(h[3]).split('.')[-2]}(%{h[1]})" for h in ins.hooks)
        return f"{r}{outs} = task {ins.name} t={ins.start}..{ins.end} ({inn}){early}"
    if isinstance(ins, Slice):
        return f"{r}%{ins.out} = slice %{ins.src} axis={ins.axis} index={ins.index}"
    if isinstance(ins, LoopIndex):
        return f"{r}%{ins.out} = loop_index {ins.index}"
    if isinstance(ins, Accum):
        k = {0: "add", 1: "concat", 2: "max"}[ins.kind]
        return f"{r}%{ins.acc} = accum.{k} %{ins.val} index={ins.index}/{ins.n}"
    if isinstance(ins, Transfer):
        vs = ", ".join(_v(values, v) for v in ins.vids)
        if view_rank is None:
            return f"{r}transfer#{ins.tid} r{ins.rank} -> r{ins.dst}: {vs}"
        if view_rank == ins.rank:
            return f"[r{view_rank}] send#{ins.tid} -> r{ins.dst}: {vs}"
        return f"[r{view_rank}] recv#{ins.tid} <- r{ins.rank}: {vs}"
    if isinstance(ins, SendDone):
        return f"{r}send_done#{ins.tid}"
    if isinstance(ins, Delete):
        return f"{r}delete " + ", ".join(f"%{v}" for v in ins.vids)
    if isinstance(ins, AllReduce):
        return f"{r}%{ins.out} = all_reduce#{ins.cid} ranks={ins.ranks} local={ins.local}"
    if isinstance(ins, AllGather):
        return f"{r}%{ins.out} = all_gather#{ins.cid} ranks={ins.ranks} axis={ins.axis} local={ins.local}"
    return f"{r}{ins}"
