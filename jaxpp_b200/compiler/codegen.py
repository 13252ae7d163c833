"""Turn a list of graph nodes into a Python callable (a *task executable*).

One executable runs one pipeline task (e.g. the forward of stage 3): it receives its inputs in a
list that it empties immediately — so inputs the caller has already dropped are freed at their
last use inside the task, the counterpart of the reference's buffer donation
(src/jaxpp/core.py:1732-1809) — runs the ops in program order, drops every intermediate after
its last use, and returns the list of outputs.  ``pp::pipeline_yield`` and ``pp::place_with``
are identities here.  Executables are cached by their generated source text, so structurally
identical stages share one (reference: the structural task cache, core.py:2256-2293).
"""
from __future__ import annotations

import operator
from typing import Any, Callable, Sequence

import torch
from torch import fx

from .. import primitives as prim


class _Consts:
    """Interning table for non-node arguments referenced from generated code."""

    def __init__(self):
        self.items: list[Any] = []
        self.keys: dict[Any, int] = {}

    def ref(self, v) -> str:
        try:
            key = (type(v).__name__, v if not isinstance(v, float) else repr(v))
            hash(key)
        except TypeError:
            key = ("id", id(v))
        if key not in self.keys:
            self.keys[key] = len(self.items)
            self.items.append(v)
        return f"C[{self.keys[key]}]"


_SIMPLE = (int, float, bool, str, type(None))
_IDENTITY_TARGETS = {torch.ops.aten.detach.default, torch.ops.aten.alias.default}


class TaskCode:
    """Source text plus the tables it refers to; ``bind(device)`` gives the callable."""

    def __init__(self, name: str, src: str, targets: list, consts: list, n_in: int, n_out: int, sink_outputs=()):
        self.name, self.src, self.targets, self.consts, self.n_in, self.n_out = name, src, targets, consts, n_in, n_out
        # output positions produced by a weight-gradient op and by nothing else: ``run(args, sink)`` accepts an
        # accumulator for them (see ops/sink.py)
        self.sink_outputs = tuple(sink_outputs)
        self._bound: dict[Any, Callable] = {}

    def key(self):
        return (self.src, tuple(id(t) for t in self.targets), tuple(repr(c) for c in self.consts))

    def bind(self, device: torch.device) -> Callable:
        from ..utils import optimes

        timed = optimes.ACTIVE[0]      # per-op timing: the same code over call targets that record CUDA events
        key = (device, timed)
        fn = self._bound.get(key)
        if fn is None:
            consts = [device if isinstance(c, torch.device) else c for c in self.consts]
            from ..ops import sink as _sink

            from ..ops import core as _ops

            # D: the implementation function of an op where one is known (called without the dispatcher), else the op
            direct = [_ops.DIRECT.get(t, t) for t in self.targets]
            targets = self.targets
            if timed:
                direct = [optimes.Timed(d, optimes.name_of(t)) for d, t in zip(direct, self.targets)]
                targets = [optimes.Timed(t) for t in self.targets]
            scope = {"T": targets, "D": direct, "C": consts, "DEV": device, "WG": _sink.call}
            exec(compile(self.src, f"<task {self.name}>", "exec"), scope)
            fn = scope["run"]
            self._bound[key] = fn
        return fn


def generate(name: str, nodes: Sequence[fx.Node], inputs: Sequence[Any], outputs: Sequence[Any],
             key_of: Callable[[fx.Node, int], Any] | None = None, members: Sequence[int] | None = None,
             attr_lookup: Callable[[str], Any] | None = None) -> TaskCode:
    """Emit code for ``nodes``.

    ``inputs``/``outputs`` are lists of *keys*; by default the key of a node is the node itself.
    For fused tasks the same node can occur once per member with different microbatches; then
    ``members[i]`` is the member index of ``nodes[i]`` and ``key_of(node, member)`` gives the key
    under which that occurrence's value is known.
    """
    if key_of is None:
        key_of = lambda n, m: n
    if members is None:
        members = [0] * len(nodes)
    mk = prim.marker_targets()
    consts = _Consts()
    targets: list[Any] = []
    target_ix: dict[int, int] = {}
    names: dict[Any, str] = {}
    lines: list[str] = []

    for i, k in enumerate(inputs):
        names[k] = f"a{i}"
    if inputs:
        lines.append(f"    {', '.join(names[k] for k in inputs)}{',' if len(inputs) == 1 else ''} = args")
    lines.append("    args.clear()")

    # last use of every key, to free values as early as possible
    last_use: dict[Any, int] = {}
    out_set = set(outputs)
    for pos, (n, m) in enumerate(zip(nodes, members)):
        for inp in n.all_input_nodes:
            last_use[key_of(inp, m)] = pos
    for k in inputs:
        if k not in last_use and k not in out_set:
            last_use[k] = -1

    def tref(t) -> str:
        if id(t) not in target_ix:
            target_ix[id(t)] = len(targets)
            targets.append(t)
        return f"T[{target_ix[id(t)]}]"

    def aref(a, m) -> str:
        if isinstance(a, fx.Node):
            return names[key_of(a, m)]
        if isinstance(a, (list, tuple)):
            inner = ", ".join(aref(x, m) for x in a)
            if isinstance(a, tuple):
                return f"({inner}{',' if len(a) == 1 else ''})"
            return f"[{inner}]"
        if isinstance(a, _SIMPLE) and not isinstance(a, float):
            return repr(a)
        if isinstance(a, slice):
            return f"slice({aref(a.start, m)}, {aref(a.stop, m)}, {aref(a.step, m)})"
        return consts.ref(a)

    from ..ops import sink as _sink

    sinkable = _sink.sink_targets()
    out_index = {}
    for j, k in enumerate(outputs):
        out_index.setdefault(k, []).append(j)
    sink_outputs: list[int] = []

    pre_free = [names[k] for k in inputs if last_use.get(k) == -1]
    if pre_free:
        lines.append(f"    {' = '.join(pre_free)} = None")

    for pos, (n, m) in enumerate(zip(nodes, members)):
        k = key_of(n, m)
        var = f"v{pos}"
        names[k] = var
        if n.op == "get_attr":
            val = attr_lookup(n.target) if attr_lookup else None
            lines.append(f"    {var} = {consts.ref(val)}.to(DEV)")
        elif n.op == "call_function":
            if n.target is mk["yield"]:
                lines.append(f"    {var} = {aref(n.args[0], m)}")
            elif n.target is mk["place_with"]:
                lines.append(f"    {var} = {aref(n.args[0], m)}")
            elif n.target is operator.getitem:
                lines.append(f"    {var} = {aref(n.args[0], m)}[{aref(n.args[1], m)}]")
            elif n.target in _IDENTITY_TARGETS:
                # an alias of its operand: tasks are functional, so the operand itself serves
                lines.append(f"    {var} = {aref(n.args[0], m)}")
            else:
                parts = [aref(a, m) for a in n.args]
                parts += [f"{kw}={aref(v, m)}" for kw, v in n.kwargs.items()]
                if n.target in sinkable and k not in last_use and len(out_index.get(k, ())) == 1:
                    # a weight gradient that only leaves the task: the caller may supply its accumulator
                    j = out_index[k][0]
                    sink_outputs.append(j)
                    lines.append(f"    {var} = WG({tref(n.target)}, sink, {j}, {', '.join(parts)})")
                elif not n.kwargs:
                    lines.append(f"    {var} = D{tref(n.target)[1:]}({', '.join(parts)})")   # implementation, no dispatcher
                else:
                    lines.append(f"    {var} = {tref(n.target)}({', '.join(parts)})")
        else:  # pragma: no cover
            raise NotImplementedError(f"cannot generate code for node {n.op}")
        dead = [kk for kk in {key_of(i, m) for i in n.all_input_nodes} if last_use.get(kk) == pos and kk not in out_set]
        if k not in last_use and k not in out_set:
            dead.append(k)
        if dead:
            lines.append(f"    {' = '.join(sorted(names[d] for d in dead))} = None")

    lines.append(f"    return [{', '.join(names[k] for k in outputs)}]")
    src = "def run(args, sink=None):\n" + "\n".join(lines) + "\n"
    return TaskCode(name, src, targets, consts.items, len(inputs), len(outputs), sink_outputs)


class CodeCache:
    """Structural cache: identical source + identical tables → one ``TaskCode``."""

    def __init__(self):
        self.table: dict[Any, TaskCode] = {}

    def intern(self, code: TaskCode) -> TaskCode:
        return self.table.setdefault(code.key(), code)
