"""Graph analyses on a captured step: dead-code removal, loop regions, stage clustering.

Behavioural counterparts in the reference (src/jaxpp/core.py): the before/loop/after split
(``wrap_into_tasks`` :1633-1729), stage clustering by backward slices of the stage markers
(``cluster_jaxpr`` :958-1031), placement of left-over loop equations by def/use
(``infer_cluster_idx_for_eqns`` :864-955), the per-stage split of gradients of shared weights
(``compute_needed`` :534-646) and the zero-bubble split of a backward cluster into its
activation-gradient and weight-gradient halves (:1075-1095, jaxpr_utils.py:105-169).
Here they operate on ``torch.fx`` nodes.
"""
from __future__ import annotations

import dataclasses
import operator
from typing import Iterable, Sequence

import torch
from torch import fx

from .. import primitives as prim
from ..types import TaskType
from ..utils import config

aten = torch.ops.aten

# ops whose result is a view/alias of an input: free to recompute, always hoisted out of the loop
_ALIAS_TARGETS = {
    aten.detach.default, aten.view.default, aten.reshape.default, aten._unsafe_view.default, aten.t.default,
    aten.transpose.int, aten.permute.default, aten.expand.default, aten.unsqueeze.default, aten.squeeze.dim,
    aten.squeeze.default, aten.alias.default, aten.slice.Tensor, aten.select.int, aten.as_strided.default,
    aten.unflatten.int, aten.flatten.using_ints,
}


def is_marker(node: fx.Node, kind: str) -> bool:
    return node.op == "call_function" and node.target is prim.marker_targets()[kind]


def dce(graph: fx.Graph) -> None:
    """Remove nodes without users (every captured op is pure; placeholders/outputs stay)."""
    for node in reversed(list(graph.nodes)):
        if node.op in ("call_function", "get_attr") and len(node.users) == 0:
            graph.erase_node(node)


def is_nondeterministic(node: fx.Node) -> bool:
    tags = getattr(node.target, "tags", ())
    return torch.Tag.nondeterministic_seeded in tags


def node_bytes(node: fx.Node) -> int:
    """Bytes of the tensor(s) a node produces (0 for non-tensor values)."""
    val = node.meta.get("val")
    vals = val if isinstance(val, (list, tuple)) else [val]
    return sum(v.numel() * v.element_size() for v in vals if isinstance(v, torch.Tensor))


_FP8_DTYPES = tuple(getattr(torch, n) for n in ("float8_e4m3fn", "float8_e5m2", "float8_e4m3fnuz", "float8_e5m2fnuz")
                    if hasattr(torch, n))


def is_fp8_cast(node: fx.Node) -> bool:
    """A conversion to an 8-bit float type.  Such casts stay next to the GEMM that consumes them (the reference keeps
    them inside the loop for the same reason, src/jaxpp/licm.py:429-452): hoisting one would keep a low-precision copy of
    every weight alive for the whole step and separate the cast from the scaling that belongs to it."""
    if node.op != "call_function" or node.target not in (aten._to_copy.default, aten.to.dtype):
        return False
    val = node.meta.get("val")
    return isinstance(val, torch.Tensor) and val.dtype in _FP8_DTYPES


# cheap ops whose result is at least as large as their operands: hoisting them out of the loop trades a small
# resident value for a large one, so with scarce memory they go back into the loop (licm.py:301-345)
_EXPANDING_TARGETS = {aten._to_copy.default, aten.to.dtype, aten.add.Tensor, aten.mul.Tensor, aten.clone.default,
                      aten.repeat.default, aten.expand_copy.default, aten.ones_like.default, aten.zeros_like.default,
                      aten.full_like.default}


_ALIASES = (aten.detach.default, aten.alias.default)


def _freeze(a):
    if isinstance(a, fx.Node):
        while a.op == "call_function" and a.target in _ALIASES:   # an alias stands for its operand (tasks are functional)
            a = a.args[0]
        return ("n", id(a))
    if isinstance(a, (list, tuple)):
        return (type(a).__name__,) + tuple(_freeze(x) for x in a)
    if isinstance(a, dict):
        return ("d",) + tuple((k, _freeze(v)) for k, v in sorted(a.items()))
    if isinstance(a, slice):
        return ("s", _freeze(a.start), _freeze(a.stop), _freeze(a.step))
    if isinstance(a, float):
        return ("f", repr(a))
    try:
        hash(a)
        return (type(a).__name__, a)
    except TypeError:
        return ("id", id(a))


def cse(graph: fx.Graph) -> int:
    """Common-subexpression elimination: a node that applies the same pure op to the same operands as an earlier one
    is replaced by it (the reference re-traces the step through a CSE trace before hoisting, src/jaxpp/licm.py:66-126).
    Stage markers, loop markers, seeded random ops and ``get_attr`` nodes are left alone.  A node of the backward pass
    is never replaced by one of the forward pass: the re-run forward of a recomputed block applies the same ops to the
    same operands as the forward pass did, and merging the two would keep every activation alive until the backward
    pass -- what recompute exists to avoid (JAX marks such blocks ``prevent_cse``; ``JAXPP_DISABLE_PREVENT_CSE`` lifts
    the barrier here as it does in the reference, src/jaxpp/core.py:3043-3074).  Returns the number of nodes removed."""
    markers = set(prim.marker_targets().values())
    seen: dict = {}
    removed = 0
    in_backward = False
    barrier = not config.disable_prevent_cse.value
    from_forward: set = set()
    for node in list(graph.nodes):
        if node.op == "call_function" and is_marker(node, "yield") and node.args[2] == prim.BWD_CODE and not in_backward:
            in_backward = True
            from_forward = set(seen.values())
        if node.op != "call_function" or node.target in markers or is_nondeterministic(node):
            continue
        schema = getattr(node.target, "_schema", None)
        if schema is not None and getattr(schema, "is_mutable", False):
            continue
        key = (id(node.target), _freeze(node.args), _freeze(node.kwargs))
        first = seen.get(key)
        if first is None or (barrier and in_backward and first in from_forward):
            seen[key] = node
            continue
        node.replace_all_uses_with(first)
        graph.erase_node(node)
        removed += 1
    return removed


@dataclasses.dataclass
class LoopRegions:
    begin: fx.Node | None
    index: fx.Node | None
    end: fx.Node
    n: int
    axis: int
    slice_of: dict  # getitem node of loop_begin → position k of the batched input
    batched_inputs: list  # loop_begin's tensor arguments
    body: list  # nodes executed per microbatch, program order
    hoisted: list  # loop-invariant nodes moved before the loop
    out_nodes: list  # loop_end operands
    out_kinds: list
    out_axes: list
    results: dict  # position k → getitem node of loop_end (if used)


def find_loop(graph: fx.Graph) -> LoopRegions | None:
    nodes = list(graph.nodes)
    pos = {n: i for i, n in enumerate(nodes)}
    ends = [n for n in nodes if is_marker(n, "loop_end")]
    begins = [n for n in nodes if is_marker(n, "loop_begin")]
    idxs = [n for n in nodes if is_marker(n, "loop_index")]
    if not ends:
        if begins or idxs:
            raise AssertionError("loop results are unused: nothing to pipeline")
        return None
    if len(ends) != 1:
        raise AssertionError(f"Exactly one treduce loop is supported, found {len(ends)}")
    end = ends[0]
    begin = begins[0] if begins else None
    index = idxs[0] if idxs else None
    start_pos = min(pos[m] for m in (begin, index) if m is not None) if (begin or index) else None
    if start_pos is None:
        raise AssertionError("loop body does not depend on the microbatch: nothing to pipeline")
    slice_of = {}
    if begin is not None:
        for u in begin.users:
            assert u.target is operator.getitem
            slice_of[u] = u.args[1]
    sources = set(slice_of) | ({index} if index is not None else set())
    between = [n for n in nodes[start_pos:pos[end]] if n is not begin and n not in sources]
    variant = set(sources)
    hoisted, body = [], []
    hoisted_set = set()
    body_set = set()
    licm = config.enable_licm.value
    for n in between:
        ins = n.all_input_nodes
        if any(i in variant for i in ins):
            variant.add(n)
            body.append(n)
            body_set.add(n)
            continue
        inputs_outside = all(i not in body_set for i in ins)
        movable = (
            inputs_outside
            and not is_marker(n, "yield")
            and not is_marker(n, "place_with")     # pins its value inside the loop (licm.py:455-456)
            and not is_nondeterministic(n)
            and not is_fp8_cast(n)
            and (licm or n.target in _ALIAS_TARGETS or n.target is operator.getitem and ins[0] in hoisted_set)
        )
        if movable:
            hoisted.append(n)
            hoisted_set.add(n)
        else:
            body.append(n)
            body_set.add(n)
    if licm and config.licm_memory_scarce.value:
        # scarce memory: a hoisted op that only expands its operands (a cast to a wider type, a broadcast add, ...)
        # and feeds nothing but the loop goes back inside, last one first, so that chains of them move together
        for n in reversed(list(hoisted)):
            if n.target not in _EXPANDING_TARGETS or not n.users:
                continue
            if not all(u in body_set for u in n.users):
                continue
            if node_bytes(n) < sum(node_bytes(i) for i in n.all_input_nodes):
                continue
            hoisted.remove(n)
            hoisted_set.discard(n)
            body_set.add(n)
        body = [n for n in between if n in body_set]
    out_nodes = list(end.args[0])
    # a microbatch slice (or the index) returned as it is: give it a node of its own in the body, so that it has a
    # producing task like every other loop output (it joins the first stage, which reads the microbatch anyway)
    if any(o in sources for o in out_nodes):
        for k, o in enumerate(out_nodes):
            if o in sources:
                with graph.inserting_before(end):
                    copy = graph.call_function(aten.clone.default, (o,))
                copy.meta.update({key: o.meta[key] for key in ("val", "tensor_meta") if key in o.meta})
                copy.meta["pp_passthrough"] = True
                out_nodes[k] = copy
                body.append(copy)
        end.args = (out_nodes, *end.args[1:])
        out_nodes = list(end.args[0])
    results = {u.args[1]: u for u in end.users}
    return LoopRegions(
        begin, index, end, end.args[3], begin.args[1] if begin is not None else 0, slice_of,
        list(begin.args[0]) if begin is not None else [], body, hoisted, out_nodes, list(end.args[1]),
        list(end.args[2]), results,
    )


@dataclasses.dataclass
class Cluster:
    stage_id: int
    task_type: TaskType
    rank: int
    nodes: list = dataclasses.field(default_factory=list)

    @property
    def name(self) -> str:
        from ..schedules import mk_task_name

        return mk_task_name(self.stage_id, self.task_type)


def _closure(targets: Iterable[fx.Node], allowed: set, assigned: dict) -> list:
    """Unassigned nodes in ``allowed`` that ``targets`` transitively depend on (incl. targets)."""
    out = []
    seen = set()
    stack = [t for t in targets]
    while stack:
        n = stack.pop()
        if n in seen or n not in allowed or n in assigned:
            continue
        seen.add(n)
        out.append(n)
        stack.extend(n.all_input_nodes)
    return out


def cluster_stages(region: Sequence[fx.Node], get_rank, mpmd_dim: int) -> tuple[list[Cluster], dict]:
    """Assign every node of ``region`` (program order) to a stage cluster.

    Returns ``(clusters, assign)`` with ``clusters[c]`` for ``c`` in ``0..2n-1`` (``n`` forward clusters by
    stage, then ``n`` backward clusters from the last stage down to stage 0; only ``n`` clusters when
    the region has no backward markers) and ``assign[node] = c``.
    """
    allowed = set(region)
    pos = {n: i for i, n in enumerate(region)}
    yields = [n for n in region if is_marker(n, "yield")]
    fwd = [y for y in yields if y.args[2] == prim.FWD_CODE]
    bwd = [y for y in yields if y.args[2] == prim.BWD_CODE]
    n = len(fwd)
    if n == 0:
        raise AssertionError("no stage markers found: call mark_stage_end at the end of every stage")
    if [y.args[1] for y in fwd] != list(range(n)):
        raise AssertionError(f"stage markers out of order: {[y.args[1] for y in fwd]}")
    has_bwd = len(bwd) > 0
    if has_bwd and [y.args[1] for y in bwd] != list(range(n - 1, -1, -1)):
        raise AssertionError(
            f"expected one backward marker per stage from {n - 1} down to 0, found {[y.args[1] for y in bwd]}"
        )
    n_clusters = 2 * n if has_bwd else n
    assign: dict = {}

    def put(nodes, c):
        for m in nodes:
            assign[m] = c

    def put_yield(y, c):
        assign[y] = c
        for u in y.users:
            assign[u] = c

    for k, y in enumerate(fwd):
        put(_closure(y.all_input_nodes, allowed, assign), k)
        put_yield(y, k + 1 if k < n - 1 else n - 1)
    for j, y in enumerate(bwd):
        put(_closure(y.all_input_nodes, allowed, assign), n - 1 if j == 0 else n + j - 1)
        put_yield(y, n + j)

    # ---- left-over nodes, pass 1: follow definitions -----------------------------------------
    # A left-over node that the program runs after a backward marker belongs to the backward pass, whatever it reads:
    # the re-run forward of a recomputed block of the FIRST stage depends on forward values and parameters only (no
    # backward marker follows it, so it is in no marker's closure), and following its definitions alone would put it
    # into the forward task -- which then runs the block twice and keeps every activation, the opposite of recompute.
    # (Only nodes that backward computations read are held back like this: what merely post-processes a forward
    # value after the markers -- the loss handed to the loop's output, say -- still follows its definitions.)
    bwd_at = [(pos[y], n + j) for j, y in enumerate(bwd)]
    needs_bwd: dict = {}    # reads, directly or not, a value of a backward cluster
    for m in region:
        needs_bwd[m] = (m in assign and assign[m] >= n) or any(needs_bwd.get(i, False) for i in m.all_input_nodes)
    feeds_bwd: dict = {}    # is read, directly or not, by such a node
    for m in reversed(region):
        feeds_bwd[m] = any(needs_bwd.get(u, False) or feeds_bwd.get(u, False) for u in m.users if u in allowed)
    floating = []
    for m in region:
        if m in assign:
            continue
        floor = None
        for p_y, c_y in bwd_at:
            if p_y < pos[m]:
                floor = c_y
        if is_marker(m, "place_with") and m.args[1] in assign:
            c = assign[m.args[1]]
        elif m.meta.get("pp_passthrough"):
            c = 0
        else:
            cs = [assign[i] for i in m.all_input_nodes if i in assign]
            c = max(cs) if cs else None
            if floor is not None and (c is None or c < floor) and has_bwd and feeds_bwd[m] and not needs_bwd[m]:
                c = floor
        if c is None:
            floating.append(m)
            continue
        put(_closure([m], allowed, assign), c)
    # ---- pass 2: follow uses -------------------------------------------------------------------
    for m in reversed(floating):
        if m in assign:
            continue
        cs = [assign[u] for u in m.users if u in assign]
        if cs:
            assign[m] = min(cs)
        elif config.conservative_loop_clustering.value:
            raise AssertionError(
                f"cannot place loop computation {m.format_node()} on a stage: it neither depends on nor feeds one"
            )
        else:
            assign[m] = n_clusters - 1
    # multi-output ops and their projections stay together
    for m in region:
        if m.target is operator.getitem and not is_marker(m.args[0], "yield") and m.args[0] in assign:
            assign[m] = assign[m.args[0]]

    clusters = []
    for c in range(n_clusters):
        stage = c if c < n else 2 * n - 1 - c
        ty = TaskType.FWD if c < n else TaskType.BWD
        clusters.append(Cluster(stage, ty, get_rank(stage)))
    for m in region:
        clusters[assign[m]].nodes.append(m)
    return clusters, assign


def _is_plain_add(n: fx.Node) -> bool:
    return (
        n.op == "call_function"
        and n.target is aten.add.Tensor
        and len(n.args) == 2
        and all(isinstance(a, fx.Node) for a in n.args)
        and n.kwargs.get("alpha", 1) == 1
        and n.args[0].meta["val"].shape == n.meta["val"].shape
        and n.args[1].meta["val"].shape == n.meta["val"].shape
    )


def split_shared_weight_grads(graph: fx.Graph, loop: LoopRegions, clusters: list[Cluster], assign: dict) -> int:
    """Give every contributing rank its own accumulator for a gradient that is summed across ranks.

    A weight used by stages on different ranks gets, from autograd, ``g = g_a + g_b`` inside the loop;
    accumulating ``g`` would move one partial gradient between ranks every microbatch.  Instead each
    partial is accumulated where it is produced and the sums are added once after the loop with a
    cross-rank ``add_multi``.  Returns the number of outputs that were split.
    """
    mk = prim.marker_targets()
    n_split = 0
    for k in range(len(loop.out_nodes)):
        if loop.out_kinds[k] != prim.OP_ADD:
            continue
        root = loop.out_nodes[k]
        if root not in assign or not _is_plain_add(root):
            continue
        leaves, internal = [], []

        def walk(n, is_root):
            if n in assign and _is_plain_add(n) and (is_root or len(n.users) == 1):
                internal.append(n)
                walk(n.args[0], False)
                walk(n.args[1], False)
            else:
                leaves.append(n)

        walk(root, True)
        if any(l not in assign for l in leaves):
            continue
        by_rank: dict[int, list] = {}
        for l in leaves:
            by_rank.setdefault(clusters[assign[l]].rank, []).append(l)
        if len(by_rank) < 2:
            continue
        n_split += 1
        partials = []
        for rank, ls in by_rank.items():
            acc = ls[0]
            c = max(assign[l] for l in ls)
            for other in ls[1:]:
                with graph.inserting_before(loop.end):
                    new = graph.call_function(aten.add.Tensor, (acc, other))
                new.meta["val"] = root.meta["val"]
                assign[new] = c
                clusters[c].nodes.append(new)
                acc = new
            partials.append(acc)
        for n in internal:
            clusters[assign[n]].nodes.remove(n)
            del assign[n]
        # rewrite loop_end: operand k ← first partial, extra operands appended
        outs = list(loop.end.args[0])
        kinds, axes = list(loop.end.args[1]), list(loop.end.args[2])
        outs[k] = partials[0]
        first_new = len(outs)
        for p in partials[1:]:
            outs.append(p)
            kinds.append(prim.OP_ADD)
            axes.append(0)
        loop.end.args = (outs, kinds, axes, loop.end.args[3])
        loop.end.meta["val"] = list(loop.end.meta["val"]) + [root.meta["val"]] * (len(partials) - 1)
        loop.out_nodes, loop.out_kinds, loop.out_axes = outs, kinds, axes
        res_k = loop.results.get(k)
        if res_k is None:
            continue
        with graph.inserting_after(res_k):
            parts = [res_k]
            anchor = res_k
            for off in range(len(partials) - 1):
                with graph.inserting_after(anchor):
                    gi = graph.call_function(operator.getitem, (loop.end, first_new + off))
                gi.meta["val"] = root.meta["val"]
                loop.results[first_new + off] = gi
                parts.append(gi)
                anchor = gi
        with graph.inserting_after(anchor):
            total = graph.call_function(mk["add_multi"], (parts,))
        total.meta["val"] = root.meta["val"]
        res_k.replace_all_uses_with(total, delete_user_cb=lambda u: u is not total)
        for n in reversed(internal):
            if len(n.users) == 0:
                graph.erase_node(n)
    return n_split


def _matmul_like(node: fx.Node) -> bool:
    """Ops that a zero-bubble split never pulls forward for free: GEMMs, attention, and the fused GEMM+collective ops."""
    name = str(node.target)
    return any(k in name for k in ("linear", "wgrad", "dgrad", "attention", "mm.", "bmm", "matmul", "ag_", "_rs"))


def split_backward_clusters(clusters: list[Cluster], assign: dict, loop_end: fx.Node | None,
                            first_stage_id: int = 0, memory_scarce: bool | None = None,
                            defer_budget_bytes: int | None = None) -> tuple[list[Cluster], dict]:
    """Zero-bubble split: each backward cluster (except the first stage's) becomes ``BWD_I`` — the
    backward slice of the values other clusters consume, i.e. the activation gradients — and
    ``BWD_W`` — everything else (weight gradients).  The first stage keeps one task typed ``BWD_I``.

    Activation recompute is traced flat (the re-run forward ops are ordinary nodes of the backward cluster), so the
    slice cuts *through* a recomputed block op by op: what the reference does by splitting a ``remat`` equation in two
    (src/jaxpp/jaxpr_utils.py:60-102).  Two refinements bound what stays alive from ``BWD_I`` to ``BWD_W``:

    * ``memory_scarce`` (default ``JAXPP_B200_ZB_MEMORY_SCARCE``, on): a left-over op that is not a GEMM, does not
      depend on a left-over GEMM and does not produce more bytes than it consumes moves into ``BWD_I`` — the smaller
      result is kept instead of its operands (jaxpr_utils.py:138-169);
    * ``defer_budget_bytes`` (default ``JAXPP_B200_ZB_DEFER_BYTES``, unlimited when negative): weight-gradient GEMMs
      are deferred to ``BWD_W`` in program order only while the operands they keep alive fit the budget; the others
      run in ``BWD_I``.  With full recompute the deferred operands (activation gradients and recomputed inputs of
      every linear) are what a zero-bubble schedule holds per outstanding microbatch, so this is the knob that makes
      a large model fit."""
    if memory_scarce is None:
        memory_scarce = config.zb_memory_scarce.value
    if defer_budget_bytes is None:
        defer_budget_bytes = config.zb_defer_bytes.value
    out: list[Cluster] = []
    new_assign: dict = {}
    for c, cl in enumerate(clusters):
        if cl.task_type is not TaskType.BWD:
            idx = len(out)
            out.append(cl)
            for m in cl.nodes:
                new_assign[m] = idx
            continue
        if cl.stage_id == first_stage_id:
            merged = Cluster(cl.stage_id, TaskType.BWD_I, cl.rank, cl.nodes)
            idx = len(out)
            out.append(merged)
            for m in cl.nodes:
                new_assign[m] = idx
            continue
        inside = set(cl.nodes)
        targets = [m for m in cl.nodes if any(u not in inside and u is not loop_end for u in m.users)]
        need = set(_closure(targets, inside, {}))
        # projections of a multi-output op stay with it
        for m in cl.nodes:
            if m.target is operator.getitem and m.args[0] in need:
                need.add(m)
        if defer_budget_bytes is not None and defer_budget_bytes >= 0:
            kept = 0
            counted: set = set()
            for m in cl.nodes:                      # program order
                if m in need or not _matmul_like(m):
                    continue
                extra = sum(node_bytes(i) for i in m.all_input_nodes if i not in counted and i.op != "placeholder")
                if kept + extra <= defer_budget_bytes:
                    kept += extra
                    counted.update(m.all_input_nodes)
                else:
                    need.update(_closure([m], inside, {}))   # runs with the activation gradients
        if memory_scarce:
            deferred_defs: set = set()
            for m in cl.nodes:                      # program order: producers before consumers
                if m in need:
                    continue
                if _matmul_like(m) or any(i in deferred_defs for i in m.all_input_nodes):
                    deferred_defs.add(m)
                    continue
                ins_bytes = sum(node_bytes(i) for i in m.all_input_nodes)
                if m.target is operator.getitem or (ins_bytes > 0 and node_bytes(m) <= ins_bytes):
                    if all(i in need or i not in inside for i in m.all_input_nodes):
                        need.add(m)
                        continue
                deferred_defs.add(m)
        part_i = Cluster(cl.stage_id, TaskType.BWD_I, cl.rank, [m for m in cl.nodes if m in need])
        part_w = Cluster(cl.stage_id, TaskType.BWD_W, cl.rank, [m for m in cl.nodes if m not in need])
        for part in (part_i, part_w):
            idx = len(out)
            out.append(part)
            for m in part.nodes:
                new_assign[m] = idx
    return out, new_assign
