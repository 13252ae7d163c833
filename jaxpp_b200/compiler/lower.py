"""Lowering of a captured step to a scheduled multi-rank program.

Pipeline (reference: src/jaxpp/core.py §"mpmdify", :2711-2896 and the passes it calls):

1. split the graph into *before-loop*, *loop body* and *after-loop* regions;
2. cluster the loop body into per-stage forward/backward tasks (``cluster.py``);
3. fully unroll the microbatch loop and list-schedule the task instances against the
   per-rank orders of the schedule (integer latencies; :1966-2098);
4. fuse the groups the schedule marks as fused into one executable (:2444-2513);
5. place before-loop computation on every rank that consumes it (replicated, never
   communicated; :1411-1445) and after-loop computation by forward propagation of placements,
   turning ``add_multi``/``gather_multi`` into cross-rank collectives (:167-466);
6. insert transfers (one per producer task and destination rank, flushed when the scheduling
   clock advances, ordered by first use; :2107-2210), ``send_done`` (:2213-2249), donation
   (:1732-1809) and deletes (:1812-1890);
7. the result is one global instruction list from which each rank takes its own part.
"""
from __future__ import annotations

import dataclasses
import math
from collections import defaultdict

from torch import fx

from .. import primitives as prim
from ..schedules import BaseSchedule, FusedTask, mk_task_name, preprocess_schedule_tasks
from ..types import TaskType
from ..utils import config, hbytes, log_elapsed_time, logger
from . import cluster as cl
from .capture import Captured
from .codegen import CodeCache, TaskCode, generate
from .program import (Accum, AllGather, AllReduce, Delete, Instr, LoopIndex, Program, RunTask, SendDone, Slice,
                      Transfer, ValueInfo)


def _meta(node: fx.Node):
    return node.meta["val"]


class _Ids:
    def __init__(self):
        self.next = 0
        self.values: dict[int, ValueInfo] = {}

    def new(self, like, label: str) -> int:
        vid = self.next
        self.next += 1
        self.values[vid] = ValueInfo(vid, tuple(like.shape), like.dtype, label)
        return vid


@dataclasses.dataclass
class _Template:
    cluster: cl.Cluster
    nodes: list
    inputs: list  # external nodes consumed (any kind)
    outputs: list  # nodes visible outside
    code: TaskCode | None = None


def _external_io(nodes: list, extra_users: set) -> tuple[list, list]:
    inside = set(nodes)
    inputs, seen = [], set()
    for n in nodes:
        for i in n.all_input_nodes:
            if i not in inside and i not in seen:
                seen.add(i)
                inputs.append(i)
    outputs = [n for n in nodes if any(u not in inside for u in n.users)]
    return inputs, outputs


class Lowering:
    def __init__(self, cap: Captured, mpmd_dim: int, name: str = "step", donated_inputs: set | None = None):
        self.donated_inputs = set(donated_inputs or ())   # positions (flat tensor inputs) the caller gave up
        self.cap = cap
        self.graph = cap.graph
        self.mpmd_dim = mpmd_dim
        self.name = name
        self.ids = _Ids()
        self.cache = CodeCache()
        self.instrs: list[Instr] = []
        self.next_tid = 0
        self.next_cid = 0
        # vid of a loop-invariant / straight-line value, per node (each rank has its own copy)
        self.const_vid: dict[fx.Node, int] = {}
        # ranks on which a vid is (or will be) materialised
        self.where: dict[int, set] = defaultdict(set)
        self.mk = prim.marker_targets()

    # ------------------------------------------------------------------------------------------
    def attr(self, target: str):
        obj = self.cap.gm
        for part in target.split("."):
            obj = getattr(obj, part)
        return obj

    def vid_of_const(self, node: fx.Node) -> int:
        v = self.const_vid.get(node)
        if v is None:
            v = self.ids.new(_meta(node), node.name)
            self.const_vid[node] = v
        return v

    def gen(self, name, nodes, inputs, outputs, **kw) -> TaskCode:
        return self.cache.intern(generate(name, nodes, inputs, outputs, attr_lookup=self.attr, **kw))

    # ------------------------------------------------------------------------------------------
    def emit_region_task(self, rank: int, name: str, nodes: list, wanted: list) -> None:
        """Emit one straight-line task on ``rank`` computing ``wanted`` from ``nodes`` (program order)."""
        if not nodes:
            return
        inside = set(nodes)
        inputs, seen = [], set()
        for n in nodes:
            for i in n.all_input_nodes:
                if i not in inside and i not in seen:
                    seen.add(i)
                    inputs.append(i)
        outputs = [n for n in nodes if n in wanted and not isinstance(_meta(n), (list, tuple))]
        code = self.gen(name, nodes, inputs, outputs)
        ins = [self.vid_of_const(i) for i in inputs]
        outs = [self.vid_of_const(o) for o in outputs]
        for v in outs:
            self.where[v].add(rank)
        self.instrs.append(RunTask(rank, name, code, ins, outs, [False] * len(ins)))

    # ------------------------------------------------------------------------------------------
    def run(self, schedule: BaseSchedule | None) -> Program:
        cap, graph = self.cap, self.graph
        cl.dce(graph)
        if config.enable_licm.value:
            n_cse = cl.cse(graph)
            if n_cse:
                logger.info("common-subexpression elimination removed %d ops", n_cse)
        if config.fuse_norm_backward_adds.value:
            from .peephole import fuse_norm_backward_adds

            fuse_norm_backward_adds(graph)
        loop = cl.find_loop(graph)
        nodes = list(graph.nodes)
        self.pos = {n: i for i, n in enumerate(nodes)}
        placeholders = cap.placeholders
        for p in placeholders:
            self.vid_of_const(p)
        flat_outputs = cap.outputs

        in_ranks: dict[fx.Node, set] = {p: set() for p in placeholders}

        if loop is not None:
            if schedule is None:
                schedule = cap.trace.schedule
            body_templates, loop_out_rank = self.lower_loop(loop, schedule, in_ranks)
            moved = self.plan_early_collectives(loop) if config.overlap_grad_reduce.value else {}
            after_exclude = set(loop.body) | set(loop.slice_of) | {loop.begin, loop.index, loop.end}
            after_exclude.discard(None)
            after_exclude |= set(loop.results.values())
            after_exclude |= set(moved)
            after_nodes = [
                n for n in graph.nodes
                if n.op in ("call_function", "get_attr") and n not in after_exclude
            ]
            fixed = {}
            for k, res in loop.results.items():
                fixed[res] = {loop_out_rank[k]}
            for node, rank in moved.items():
                fixed[node] = {rank}
            self.lower_straight(after_nodes, fixed, in_ranks, flat_outputs, label="after_loop")
        else:
            region = [n for n in graph.nodes if n.op in ("call_function", "get_attr")]
            self.lower_by_yield(region, in_ranks, flat_outputs)

        # ---- program inputs / outputs ------------------------------------------------------
        inputs = []
        for p in placeholders:
            ranks = tuple(sorted(in_ranks[p]))
            inputs.append((self.const_vid[p], ranks))
            for r in ranks or (0,):
                self.where[self.const_vid[p]].add(r)
        outputs = []
        for o in flat_outputs:
            if isinstance(o, fx.Node):
                vid = self.const_vid[o]
                outputs.append(("v", vid, tuple(sorted(self.where[vid]))))
            else:
                outputs.append(("c", o))
        # program inputs stay alive for the whole step unless the caller donated them: a donated input is freed
        # after its last use on each rank like any intermediate (reference: infer_donation, core.py:1732-1809)
        self.finish_lifetimes({v for kind, v, *_ in [o for o in outputs if o[0] == "v"]},
                              {vid for k, (vid, _) in enumerate(inputs) if k not in self.donated_inputs})
        prog = Program(self.mpmd_dim, self.instrs, self.ids.values, inputs, outputs)
        prog.meta["name"] = self.name
        prog.meta["n_mubatches"] = loop.n if loop is not None else 1
        prog.meta["schedule"] = repr(schedule) if schedule is not None else None
        if config.enable_check_ir.value:
            from .verify import verify_program

            verify_program(prog)
        return prog

    # ==========================================================================================
    # loop
    # ==========================================================================================
    def lower_loop(self, loop: cl.LoopRegions, schedule: BaseSchedule, in_ranks):
        graph = self.graph
        n_mb = loop.n
        if schedule is None:
            raise AssertionError("treduce needs a schedule")
        clusters, assign = cl.cluster_stages(loop.body, schedule.get_mpmd_idx, self.mpmd_dim)
        n_stages = len([c for c in clusters if c.task_type is TaskType.FWD])
        if not any(c.task_type is TaskType.BWD for c in clusters):
            raise AssertionError(
                "the loop body has no backward pass; use mpmd_jit_by_yield for forward-only pipelines"
            )
        if n_stages != schedule.num_stages:
            raise AssertionError(
                f"the loop body marks {n_stages} stages but the schedule was built for {schedule.num_stages}"
            )
        for c in clusters:
            if not 0 <= c.rank < self.mpmd_dim:
                raise AssertionError(f"stage {c.stage_id} maps to rank {c.rank} outside a mesh of {self.mpmd_dim}")
        n_split = cl.split_shared_weight_grads(graph, loop, clusters, assign)
        if n_split:
            logger.info("split %d cross-rank gradient sums into per-rank accumulators", n_split)
        if schedule.is_partial_bwd:
            clusters, assign = cl.split_backward_clusters(clusters, assign, loop.end)
        self.pos = {n: i for i, n in enumerate(graph.nodes)}
        for c in clusters:
            c.nodes.sort(key=self.pos.__getitem__)

        body_set = set(assign)
        sources = set(loop.slice_of) | ({loop.index} if loop.index is not None else set())
        templates: dict[tuple[int, TaskType], _Template] = {}
        def_template: dict[fx.Node, _Template] = {}
        for c in clusters:
            inputs, outputs = _external_io(c.nodes, set())
            outputs = [o for o in outputs if not isinstance(_meta(o), (list, tuple))]
            t = _Template(c, c.nodes, inputs, outputs)
            templates[(c.stage_id, c.task_type)] = t
            for m in c.nodes:
                def_template[m] = t
        for t in templates.values():
            for i in t.inputs:
                if i in body_set and isinstance(_meta(i), (list, tuple)):
                    raise AssertionError(f"multi-output value {i} crosses a task boundary")

        # ---- activation size log (reference: core.py:1115) -------------------------------------
        for t in templates.values():
            nbytes = sum(_meta(o).numel() * _meta(o).element_size() for o in t.outputs)
            logger.info("task %s: %d ops, outputs %s", t.cluster.name, len(t.nodes), hbytes(nbytes))

        # ---- before-loop: replicate loop-invariant compute on every consumer rank ---------------
        consts_by_rank: dict[int, list] = defaultdict(list)
        for t in templates.values():
            for i in t.inputs:
                if i in body_set or i in sources:
                    if i in loop.slice_of:
                        consts_by_rank[t.cluster.rank].append(loop.batched_inputs[loop.slice_of[i]])
                    continue
                consts_by_rank[t.cluster.rank].append(i)
        n_before_total = 0
        for rank in range(self.mpmd_dim):
            wanted = consts_by_rank.get(rank, [])
            need, stack = set(), list(wanted)
            while stack:
                m = stack.pop()
                if m in need:
                    continue
                need.add(m)
                if m.op == "placeholder":
                    in_ranks[m].add(rank)
                    continue
                stack.extend(m.all_input_nodes)
            compute = sorted((m for m in need if m.op != "placeholder"), key=self.pos.__getitem__)
            n_before_total += len(compute)
            self.emit_region_task(rank, f"before_loop_r{rank}", compute, set(wanted))
        distinct = len({m for r in consts_by_rank for m in consts_by_rank[r] if m.op != "placeholder"})
        if distinct:
            logger.info("before-loop replication factor %.2f", n_before_total / max(1, distinct))

        # ---- unroll + list scheduling ----------------------------------------------------------------
        sched_lists = preprocess_schedule_tasks(
            schedule.tasks(n_mb), first_stage_id=0, unpack_fused_tasks=config.disable_schedule_task_fusion.value
        )
        if len(sched_lists) != self.mpmd_dim:
            raise AssertionError(
                f"the schedule drives {len(sched_lists)} pipeline ranks but the mesh has {self.mpmd_dim}"
            )
        deps: dict[tuple, list] = {}
        for key, t in templates.items():
            deps[key] = sorted(
                {(def_template[i].cluster.stage_id, def_template[i].cluster.task_type) for i in t.inputs if i in body_set},
                key=lambda k: (k[0], k[1].value),
            )
        units = self.list_schedule(sched_lists, templates, deps, n_mb)

        # ---- emission ------------------------------------------------------------------------------
        body_vid: dict[tuple, int] = {}
        slice_vid: dict[tuple, int] = {}
        index_vid: dict[tuple, int] = {}
        acc_vid = {}
        loop_out_rank = {}
        out_positions: dict[fx.Node, list] = defaultdict(list)
        for k, o in enumerate(loop.out_nodes):
            out_positions[o].append(k)
            if o not in def_template:
                raise AssertionError(f"loop output {k} does not depend on the microbatch")
            loop_out_rank[k] = def_template[o].cluster.rank
            like = self.graph_val(loop.end, k)
            res = loop.results.get(k)
            if res is not None:
                acc_vid[k] = self.vid_of_const(res)
            else:
                acc_vid[k] = self.ids.new(like, f"acc{k}")
            self.where[acc_vid[k]].add(loop_out_rank[k])

        # consumers on other ranks, per produced node
        remote_users: dict[fx.Node, set] = defaultdict(set)
        for t in templates.values():
            for i in t.inputs:
                if i in body_set and def_template[i].cluster.rank != t.cluster.rank:
                    remote_users[i].add(t.cluster.rank)
        unit_order = {id(u): k for k, u in enumerate(units)}
        first_use: dict[tuple, int] = {}
        for k, u in enumerate(units):
            for (t, mb) in u.members:
                for i in t.inputs:
                    if i in body_set:
                        first_use.setdefault((i, mb, t.cluster.rank), k)

        pending: list[tuple] = []  # (first use, src, dst, vids)
        cur_time = None

        def flush():
            pending.sort(key=lambda p: (p[0], p[1], p[2]))
            for _, src, dst, vids in pending:
                self.instrs.append(Transfer(src, dst, vids, self.next_tid))
                self.next_tid += 1
                for v in vids:
                    self.where[v].add(dst)
            pending.clear()

        single_use_outputs = {o for o in loop.out_nodes if all(u is loop.end for u in o.users)}
        for u in units:
            if cur_time is not None and u.start != cur_time:
                flush()
            cur_time = u.start
            rank = u.rank
            # inputs
            produced_inside = set()
            keys_in: list = []
            vids_in: list[int] = []

            def key_for(node, mb):
                return (node, mb) if (node in body_set or node in sources) else (node, None)

            for (t, mb) in u.members:
                for i in t.inputs:
                    k = key_for(i, mb)
                    if k in produced_inside or k in keys_in:
                        continue
                    if i in loop.slice_of:
                        sk = (loop.slice_of[i], mb, rank)
                        if sk not in slice_vid:
                            v = self.ids.new(_meta(i), f"{i.name}@{mb}")
                            slice_vid[sk] = v
                            src = self.const_vid[loop.batched_inputs[loop.slice_of[i]]]
                            self.instrs.append(Slice(rank, v, src, loop.axis, mb))
                            self.where[v].add(rank)
                        vid = slice_vid[sk]
                    elif i is loop.index:
                        ik = (mb, rank)
                        if ik not in index_vid:
                            v = self.ids.new(_meta(i), f"i@{mb}")
                            index_vid[ik] = v
                            self.instrs.append(LoopIndex(rank, v, mb))
                            self.where[v].add(rank)
                        vid = index_vid[ik]
                    elif i in body_set:
                        vid = body_vid[(i, mb)]
                    else:
                        vid = self.const_vid[i]
                    keys_in.append(k)
                    vids_in.append(vid)
                for m in t.nodes:
                    produced_inside.add((m, mb))
            # outputs: everything a member exposes that someone outside this unit consumes
            member_set = {(id(t), mb) for t, mb in u.members}
            keys_out, vids_out = [], []
            for (t, mb) in u.members:
                for o in t.outputs:
                    used_outside = False
                    for usr in o.users:
                        if usr is loop.end:
                            used_outside = True
                        elif usr in def_template and (id(def_template[usr]), mb) not in member_set:
                            used_outside = True
                    if not used_outside:
                        continue
                    v = self.ids.new(_meta(o), f"{o.name}@{mb}")
                    body_vid[(o, mb)] = v
                    self.where[v].add(rank)
                    keys_out.append((o, mb))
                    vids_out.append(v)
            if len(u.members) == 1:
                t, mb = u.members[0]
                if t.code is None:
                    t.code = self.gen(t.cluster.name, t.nodes, t.inputs, t.outputs)
                # a template's code exposes all of its outputs; map the ones nobody needs to fresh ids
                code = t.code
                ins = []
                for i in t.inputs:
                    ins.append(vids_in[keys_in.index(key_for(i, mb))])
                outs = []
                for o in t.outputs:
                    if (o, mb) in body_vid and (o, mb) in keys_out:
                        outs.append(body_vid[(o, mb)])
                    else:
                        outs.append(-1)
                name = mk_task_name(t.cluster.stage_id, t.cluster.task_type, mb)
                self.instrs.append(RunTask(rank, name, code, ins, outs, [False] * len(ins), t.cluster.stage_id,
                                           t.cluster.task_type, mb, u.start, u.end))
            else:
                all_nodes, member_ix = [], []
                for mi, (t, mb) in enumerate(u.members):
                    all_nodes.extend(t.nodes)
                    member_ix.extend([mi] * len(t.nodes))
                mbs = [mb for _, mb in u.members]
                # keys relative to the first member's microbatch so that the code is reusable
                base = mbs[0]

                def rel(k):
                    node, mb = k
                    return (node, None if mb is None else mb - base)

                code = self.gen(
                    "fused_" + "_".join(t.cluster.name for t, _ in u.members),
                    all_nodes, [rel(k) for k in keys_in], [rel(k) for k in keys_out],
                    key_of=lambda node, mi: rel(key_for(node, mbs[mi])), members=member_ix,
                )
                name = "fused_" + "_".join(mk_task_name(t.cluster.stage_id, t.cluster.task_type, mb) for t, mb in u.members)
                self.instrs.append(RunTask(rank, name, code, vids_in, vids_out, [False] * len(vids_in),
                                           u.members[0][0].cluster.stage_id, None, mbs[0], u.start, u.end))
            # accumulate loop outputs, queue transfers
            by_dst: dict[int, list] = defaultdict(list)
            task = self.instrs[-1]
            for (o, mb), v in zip(keys_out, vids_out):
                for k in out_positions.get(o, ()):
                    steal = o in single_use_outputs and len(out_positions[o]) == 1
                    if (steal and loop.out_kinds[k] == 0 and config.wgrad_sinks.value and not remote_users.get(o)
                            and v in task.outs and task.outs.index(v) in task.code.sink_outputs):
                        task.sinks.append((task.outs.index(v), acc_vid[k]))
                    self.instrs.append(Accum(rank, acc_vid[k], v, loop.out_kinds[k], loop.out_axes[k], mb, n_mb, steal))
                for dst in sorted(remote_users.get(o, ())):
                    by_dst[dst].append(((o, mb), v))
            for dst, items in by_dst.items():
                fu = min(first_use.get((o, mb, dst), math.inf) for (o, mb), _ in items)
                pending.append((fu, rank, dst, [v for _, v in items]))
        flush()
        self.units = units
        self.acc_vid = acc_vid
        return templates, loop_out_rank

    # ------------------------------------------------------------------------------------------
    def plan_early_collectives(self, loop) -> dict:
        """Move gradient collectives from after the loop into the backward pass of the last microbatch.

        A step sums every weight gradient over the microbatches (``treduce``) and then, after the loop, reduces it
        over the data-parallel ranks (``b200tp::all_reduce``, or ``b200dp::reduce_scatter_flat`` with sharded
        optimizer state).  When the accumulator is fed through a weight-gradient sink, the task that adds the
        *last* contribution is known here, and so is the moment inside it when the gradient is final: right after
        that weight-gradient GEMM.  The collective is attached to the task as a hook; the executor issues it at
        that point on a side stream, where it overlaps the rest of the backward pass (earlier layers' gradients,
        other stages' tasks), and the after-loop region reads its result instead of running it.  The reference gets
        the same overlap from XLA's latency-hiding scheduler over its after-loop reduce-scatter (PERF_GUIDE.md:63-70).
        Same kernels, same operands: the results are bit-identical to the after-loop form.

        Returns ``{after-loop collective node: pipeline rank}`` for the nodes that were moved."""
        from ..ops.sink import early_collective_targets

        targets = early_collective_targets()
        moved: dict = {}
        if loop.n < 2:
            return moved
        for k, res in loop.results.items():
            if loop.out_kinds[k] != prim.OP_ADD or k not in self.acc_vid:
                continue
            users = list(res.users)
            if len(users) != 1 or users[0].target not in targets or users[0].args[0] is not res:
                continue
            node = users[0]
            if any(isinstance(a, fx.Node) for a in node.args[1:]) or node.kwargs:
                continue
            acc = self.acc_vid[k]
            last_task = None
            last_acc = None
            for ins in self.instrs:
                if isinstance(ins, RunTask) and any(a == acc for _, a in ins.sinks):
                    last_task = ins
                elif isinstance(ins, Accum) and ins.acc == acc:
                    last_acc = ins
            if last_task is None or last_acc is None:
                continue
            pos = next(j for j, a in last_task.sinks if a == acc)
            if last_task.outs[pos] != last_acc.val:
                continue   # the final contribution does not come through the sink
            result = self.vid_of_const(node)
            last_task.hooks.append((pos, acc, result, node.target, tuple(node.args[1:])))
            self.where[result].add(last_task.rank)
            moved[node] = last_task.rank
        if moved:
            logger.info("%d gradient collectives issued from the last microbatch's backward tasks", len(moved))
        return moved

    def graph_val(self, node: fx.Node, k: int):
        return _meta(node)[k]

    # ------------------------------------------------------------------------------------------
    def list_schedule(self, sched_lists, templates, deps, n_mb):
        """Order the unrolled tasks: repeatedly start, among the ranks whose next scheduled unit has
        all its dependencies done, the one that can start earliest (ties: lowest rank)."""

        @dataclasses.dataclass
        class Unit:
            rank: int
            members: list
            start: int = 0
            end: int = 0

        done: dict[tuple, int] = {}
        cursor = [0] * len(sched_lists)
        clock = [0] * len(sched_lists)
        units = []
        total = sum(len(ts) for ts in sched_lists)
        seen_keys = set()
        while len(units) < total:
            best = None
            for r, ts in enumerate(sched_lists):
                if cursor[r] >= len(ts):
                    continue
                entry = ts[cursor[r]]
                members = list(entry) if isinstance(entry, FusedTask) else [entry]
                ready, ok, inside = clock[r], True, set()
                for t in members:
                    key = (t.stage_id, t.fwd_or_bwd)
                    if key not in templates:
                        raise AssertionError(
                            f"the schedule contains {t} but the loop body has no such task "
                            f"(available: {sorted(str(mk_task_name(s, ty)) for s, ty in templates)})"
                        )
                    if templates[key].cluster.rank != r:
                        raise AssertionError(f"schedule runs {t} on rank {r} but stage {t.stage_id} lives on rank "
                                             f"{templates[key].cluster.rank}")
                    for d in deps[key]:
                        dk = (d[0], d[1], t.mubatch_idx)
                        if dk in inside:
                            continue
                        if dk not in done:
                            ok = False
                            break
                        ready = max(ready, done[dk])
                    if not ok:
                        break
                    inside.add((t.stage_id, t.fwd_or_bwd, t.mubatch_idx))
                if ok and (best is None or ready < best[0]):
                    best = (ready, r, members)
            if best is None:
                stuck = [str(ts[cursor[r]]) for r, ts in enumerate(sched_lists) if cursor[r] < len(ts)]
                raise AssertionError(f"Schedule does not honor data dependencies; blocked at {stuck}")
            start, r, members = best
            end = start + sum(t.latency for t in members)
            for t in members:
                k = (t.stage_id, t.fwd_or_bwd, t.mubatch_idx)
                if k in seen_keys:
                    raise AssertionError(f"schedule runs {t} twice")
                seen_keys.add(k)
                done[k] = end
            clock[r] = end
            cursor[r] += 1
            units.append(Unit(r, [(templates[(t.stage_id, t.fwd_or_bwd)], t.mubatch_idx) for t in members], start, end))
        expected = {(s, ty, m) for (s, ty) in templates for m in range(n_mb)}
        if seen_keys != expected:
            missing = sorted(mk_task_name(s, ty, m) for s, ty, m in expected - seen_keys)
            raise AssertionError(f"Loop tasks missing from the schedule: {missing[:8]}{'…' if len(missing) > 8 else ''}")
        units.sort(key=lambda u: (u.start, u.end, u.rank))
        return units

    # ==========================================================================================
    # straight-line regions (after the loop)
    # ==========================================================================================
    def lower_straight(self, region: list, fixed: dict, in_ranks: dict, flat_outputs: list, label: str):
        """Place ``region`` (program order) by forward propagation of placement sets.

        ``fixed`` gives the placement of values defined elsewhere (loop results).  A value whose
        operands share no rank must come from ``add_multi`` / ``gather_multi`` — these become
        collectives; anything else is an error (the computation cannot be replicated).
        """
        mk = self.mk
        all_ranks = set(range(self.mpmd_dim))
        region_set = set(region)
        out_nodes = [o for o in flat_outputs if isinstance(o, fx.Node)]
        # keep only what the outputs need
        need, stack = set(), list(out_nodes)
        while stack:
            m = stack.pop()
            if m in need:
                continue
            need.add(m)
            if m in region_set:
                stack.extend(m.all_input_nodes)
        region = [m for m in region if m in need]

        place: dict[fx.Node, set | None] = dict(fixed)

        def placement_of(m):
            if m in place:
                return place[m]
            if m.op == "placeholder":
                return set(in_ranks[m]) if in_ranks[m] else None
            if m in self.const_vid and self.where[self.const_vid[m]]:
                return set(self.where[self.const_vid[m]])
            return None

        collectives = {}
        for m in region:
            sets = [placement_of(i) for i in m.all_input_nodes]
            known = [s for s in sets if s is not None]
            if m.target is mk["add_multi"] or m.target is mk["gather_multi"]:
                operands = list(m.args[0])
                op_sets = [placement_of(o) for o in operands]
                if all(s is None for s in op_sets):
                    place[m] = None
                    continue
                inter = set.intersection(*[s for s in op_sets if s is not None])
                if inter:
                    place[m] = inter  # everything is already together: plain local op
                    continue
                owners = [min(s) if s is not None else None for s in op_sets]
                ranks = sorted({r for s in op_sets if s is not None for r in s})
                owners = [o if o is not None else ranks[0] for o in owners]
                collectives[m] = (ranks, owners)
                place[m] = set(ranks)
                continue
            if not known:
                place[m] = None
                continue
            inter = set.intersection(*known)
            if not inter:
                raise AssertionError(
                    f"After loop computation is not replicateable: {m.format_node()} combines values living on "
                    f"disjoint pipeline ranks {known}; use cross_mpmd_all_reduce / cross_mpmd_stack"
                )
            place[m] = inter

        # ranks on which each node must actually run: walk uses backwards
        run_on: dict[fx.Node, set] = defaultdict(set)
        for o in out_nodes:
            p = placement_of(o)
            run_on[o] |= (p if p is not None else all_ranks)
        for m in reversed(region):
            p = place[m]
            ranks = run_on[m] if p is None else (run_on[m] & p if m not in collectives else set(p))
            if m in collectives:
                ranks = set(collectives[m][0])
            run_on[m] = ranks
            if m in collectives:
                cranks, owners = collectives[m]
                for o, owner in zip(m.args[0], owners):
                    run_on[o].add(owner)
                continue
            for i in m.all_input_nodes:
                run_on[i] |= ranks
        for p in self.cap.placeholders:
            if p in run_on:
                in_ranks[p] |= run_on[p]

        # emit: per-rank open segments, closed at collectives and at the end
        open_seg: dict[int, list] = defaultdict(list)
        seg_count = defaultdict(int)

        def close(rank):
            nodes = open_seg[rank]
            if not nodes:
                return
            inside = set(nodes)
            wanted = {m for m in nodes if m in out_nodes or any(u not in inside and u in need for u in m.users)}
            self.emit_region_task(rank, f"{label}_r{rank}_{seg_count[rank]}", nodes, wanted)
            seg_count[rank] += 1
            open_seg[rank] = []

        for m in region:
            if m in collectives:
                ranks, owners = collectives[m]
                for r in ranks:
                    close(r)
                out = self.vid_of_const(m)
                cid = self.next_cid
                self.next_cid += 1
                operands = list(m.args[0])
                if m.target is mk["add_multi"]:
                    for r in ranks:
                        local = [self.const_vid[o] for o, owner in zip(operands, owners) if owner == r]
                        self.instrs.append(AllReduce(r, list(ranks), local, out, cid))
                        self.where[out].add(r)
                else:
                    for r in ranks:
                        local = {p: self.const_vid[o] for p, (o, owner) in enumerate(zip(operands, owners)) if owner == r}
                        self.instrs.append(AllGather(r, list(ranks), local, list(owners), m.args[1], out, cid))
                        self.where[out].add(r)
                continue
            for r in sorted(run_on[m]):
                open_seg[r].append(m)
        for r in sorted(open_seg):
            close(r)
        for o in out_nodes:
            v = self.vid_of_const(o)
            if o.op == "placeholder":
                # passthrough output: lives wherever the input lives
                if not in_ranks[o]:
                    in_ranks[o].add(0)
                self.where[v] |= in_ranks[o]

    # ==========================================================================================
    # no loop: tasks are the stages themselves, run in order (mpmd_jit_by_yield)
    # ==========================================================================================
    def lower_by_yield(self, region: list, in_ranks: dict, flat_outputs: list):
        """Forward (or forward+backward) pipeline without a microbatch loop: stage ``s`` runs on rank
        ``s % mpmd_dim`` (reference: core.py:3120-3148)."""
        get_rank = lambda s: s % self.mpmd_dim
        prev = config.conservative_loop_clustering
        with prev.set(False):
            clusters, assign = cl.cluster_stages(region, get_rank, self.mpmd_dim)
        out_nodes = {o for o in flat_outputs if isinstance(o, fx.Node)}
        done_on: dict[fx.Node, set] = defaultdict(set)
        for c in clusters:
            nodes = c.nodes
            if not nodes:
                continue
            inside = set(nodes)
            rank = c.rank
            # bring remote inputs over
            by_src: dict[int, list] = defaultdict(list)
            for m in nodes:
                for i in m.all_input_nodes:
                    if i in inside:
                        continue
                    if i.op == "placeholder":
                        in_ranks[i].add(rank)
                        continue
                    if rank not in done_on[i]:
                        src = min(done_on[i])
                        if self.const_vid[i] not in by_src[src]:
                            by_src[src].append(self.const_vid[i])
                        done_on[i].add(rank)
            for src, vids in sorted(by_src.items()):
                self.instrs.append(Transfer(src, rank, vids, self.next_tid))
                self.next_tid += 1
                for v in vids:
                    self.where[v].add(rank)
            wanted = {m for m in nodes if m in out_nodes or any(u not in inside for u in m.users)}
            wanted = {m for m in wanted if not isinstance(_meta(m), (list, tuple))}
            self.emit_region_task(rank, c.name, nodes, wanted)
            for m in wanted:
                done_on[m].add(rank)
        for o in out_nodes:
            v = self.vid_of_const(o)
            if o.op == "placeholder":
                if not in_ranks[o]:
                    in_ranks[o].add(0)
                self.where[v] |= in_ranks[o]

    # ==========================================================================================
    # lifetimes: send_done, donation, deletes
    # ==========================================================================================
    def finish_lifetimes(self, output_vids: set, input_vids: set):
        instrs = self.instrs
        # send_done: after `delay` later sends on the same channel, else at the end of the program
        delay = config.transfer_done_delay.value
        tail: list[Instr] = []
        if delay == math.inf:
            for ins in instrs:
                if isinstance(ins, Transfer):
                    tail.append(SendDone(ins.rank, ins.tid))
            instrs = instrs + tail
        else:
            out: list[Instr] = []
            inflight: dict[tuple, list] = defaultdict(list)
            for ins in instrs:
                out.append(ins)
                if isinstance(ins, Transfer):
                    ch = (ins.rank, ins.dst)
                    inflight[ch].append(ins.tid)
                    while len(inflight[ch]) > delay:
                        out.append(SendDone(ins.rank, inflight[ch].pop(0)))
            for ch, tids in inflight.items():
                for tid in tids:
                    out.append(SendDone(ch[0], tid))
            instrs = out

        # last use of each value on each rank
        last: dict[tuple, int] = {}

        def uses(ins):
            if isinstance(ins, RunTask):
                return [(ins.rank, v) for v in ins.ins]
            if isinstance(ins, Slice):
                return [(ins.rank, ins.src)]
            if isinstance(ins, Accum):
                return [(ins.rank, ins.val), (ins.rank, ins.acc)]
            if isinstance(ins, Transfer):
                return [(ins.rank, v) for v in ins.vids]
            if isinstance(ins, AllReduce):
                return [(ins.rank, v) for v in ins.local]
            if isinstance(ins, AllGather):
                return [(ins.rank, v) for v in ins.local.values()]
            return []

        def defs(ins):
            if isinstance(ins, RunTask):
                return [(ins.rank, v) for v in ins.outs if v >= 0] + [(ins.rank, h[2]) for h in ins.hooks]
            if isinstance(ins, (Slice, LoopIndex)):
                return [(ins.rank, ins.out)]
            if isinstance(ins, Transfer):
                return [(ins.dst, v) for v in ins.vids]
            if isinstance(ins, (AllReduce, AllGather)):
                return [(ins.rank, ins.out)]
            return []

        for k, ins in enumerate(instrs):
            for key in uses(ins):
                last[key] = k
            for key in defs(ins):
                last.setdefault(key, k)
        keep = output_vids | input_vids
        final: list[Instr] = []
        for k, ins in enumerate(instrs):
            if isinstance(ins, RunTask):
                ins.donate = [last[(ins.rank, v)] == k and v not in keep and ins.ins.count(v) == 1 for v in ins.ins]
            final.append(ins)
            dead = defaultdict(list)
            for (rank, v) in dict.fromkeys(uses(ins) + defs(ins)):
                if last.get((rank, v)) == k and v not in keep:
                    if isinstance(ins, RunTask) and rank == ins.rank and v in ins.ins and ins.donate[ins.ins.index(v)]:
                        continue  # already dropped by donation
                    dead[rank].append(v)
            for rank, vids in dead.items():
                final.append(Delete(rank, vids))
        self.instrs = final


def lower(cap: Captured, mpmd_dim: int, schedule: BaseSchedule | None = None, name: str = "step",
          donated_inputs: set | None = None) -> Program:
    with log_elapsed_time("compile/lower"):
        return Lowering(cap, mpmd_dim, name, donated_inputs).run(schedule)
