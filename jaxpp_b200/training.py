"""``treduce``: the pipelined microbatch loop (reference: src/jaxpp/training.py:106-340).

``treduce(fun, xs, schedule)`` applies ``fun`` to every slice ``xs[i]`` along ``axis`` and
combines the results leaf by leaf with an accumulation op: :data:`Add` (sum), :data:`Max`
(element-wise maximum) or :class:`Concat` (stack along a new axis).  The default
``(Concat(), Add)`` stacks the first output (losses / aux) and sums the second (gradients).

Run eagerly it *is* that sequential loop — this is the un-pipelined oracle.  Inside
``mpmd_jit_with_loop`` the body is captured once between ``pp::loop_begin`` and
``pp::loop_end`` markers and the compiler unrolls it against ``schedule``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable

import torch
from torch.utils import _pytree as pytree

from .primitives import OP_ADD, OP_CONCAT, OP_MAX, current_trace
from .schedules import BaseSchedule

__all__ = ["treduce", "treduce_i", "take", "Add", "Max", "Concat", "AddT", "MaxT", "default_op"]


def take(x: torch.Tensor, i, axis: int = 0) -> torch.Tensor:
    """``x`` sliced at index ``i`` along ``axis``; ``i`` may be a Python int or the 0-d index tensor
    that :func:`treduce_i` passes to its body while a step is being captured."""
    if isinstance(i, torch.Tensor):
        return x.index_select(axis, i.reshape(1)).squeeze(axis)
    return x.select(axis, i)


@dataclasses.dataclass(frozen=True)
class AddT:
    """Element-wise sum over microbatches."""

    code = OP_ADD
    axis = 0

    def state(self, n: int, a: torch.Tensor) -> torch.Tensor:
        return torch.zeros_like(a)

    def update(self, state, update, index):
        return state + update


@dataclasses.dataclass(frozen=True)
class MaxT:
    """Element-wise maximum over microbatches."""

    code = OP_MAX
    axis = 0

    def state(self, n: int, a: torch.Tensor) -> torch.Tensor:
        lo = float("-inf") if a.dtype.is_floating_point else torch.iinfo(a.dtype).min
        return torch.full_like(a, lo)

    def update(self, state, update, index):
        return torch.maximum(state, update)


@dataclasses.dataclass(frozen=True)
class Concat:
    """Stack per-microbatch values along a new axis at position ``axis``."""

    axis: int = 0
    code = OP_CONCAT

    def state(self, n: int, a: torch.Tensor) -> torch.Tensor:
        assert n > 0
        shape = list(a.shape)
        shape.insert(self.axis, n)
        return a.new_zeros(shape)

    def update(self, state, update, index):
        out = state.clone()
        out.select(self.axis, index).copy_(update)
        return out


Add = AddT()
Max = MaxT()
default_op = (Concat(), Add)


def _is_op(x) -> bool:
    return isinstance(x, (AddT, MaxT, Concat))


def _broadcast_ops(operation, out_tree_example):
    """Prefix-broadcast ``operation`` over the structure of the body's output."""

    def expand(op, sub):
        if _is_op(op):
            return [op] * len(pytree.tree_leaves(sub))
        if isinstance(op, (tuple, list)):
            if not isinstance(sub, (tuple, list)) or len(sub) != len(op):
                raise ValueError(f"`operation` {op} does not match the structure of the loop output")
            return [o for a, b in zip(op, sub) for o in expand(a, b)]
        if isinstance(op, dict):
            if not isinstance(sub, dict) or set(op) != set(sub):
                raise ValueError(f"`operation` {op} does not match the structure of the loop output")
            # pytree flattens dicts in insertion order of ``sub``
            return [o for k in sub for o in expand(op[k], sub[k])]
        raise TypeError(f"unsupported accumulation op {op!r}")

    return expand(operation, out_tree_example)


def treduce(fun: Callable, xs: Any, schedule: BaseSchedule, axis: int = 0, operation=default_op) -> Any:
    leaves, spec = pytree.tree_flatten(xs)
    if not leaves:
        raise ValueError("treduce needs at least one batched input")
    n = leaves[0].shape[axis]
    if any(l.shape[axis] != n for l in leaves):
        raise AssertionError("Leading dimensions differing among xs")

    ctx = current_trace()
    if ctx is None:  # eager: the sequential oracle
        def body(i):
            return fun(pytree.tree_unflatten([l.select(axis, i) for l in leaves], spec))

        return _sequential(body, n, operation)

    _enter_loop(ctx, schedule, n)
    slices = torch.ops.pp.loop_begin(list(leaves), axis, n)
    out = fun(pytree.tree_unflatten(list(slices), spec))
    return _close_loop(ctx, out, operation, n)


def treduce_i(fun: Callable[[Any], Any], length: int, schedule: BaseSchedule, operation=default_op) -> Any:
    """Like :func:`treduce` but ``fun`` receives the microbatch index (a 0-d int64 tensor under
    capture, a Python int when run eagerly) instead of a slice."""
    ctx = current_trace()
    if ctx is None:
        return _sequential(fun, length, operation)
    _enter_loop(ctx, schedule, length)
    device = _TRACE_DEVICE[-1] if _TRACE_DEVICE else torch.device("cpu")
    idx = torch.ops.pp.loop_index(length, device)
    out = fun(idx)
    return _close_loop(ctx, out, operation, length)


_TRACE_DEVICE: list[torch.device] = []


def _enter_loop(ctx, schedule, n):
    if ctx.n_loops >= 1:
        raise AssertionError("Only one treduce loop is supported per mpmd_jit_with_loop function")
    ctx.n_loops += 1
    ctx.schedule = schedule
    ctx.n_mubatches = n
    ctx.in_loop = True
    ctx.stage_counter = 0  # stage ids count from the start of the loop body


def _close_loop(ctx, out, operation, n):
    out_leaves, out_spec = pytree.tree_flatten(out)
    ops = _broadcast_ops(operation, out)
    if len(ops) != len(out_leaves):
        raise ValueError("`operation` does not match the structure of the loop output")
    res = torch.ops.pp.loop_end(
        [o.contiguous() for o in out_leaves], [op.code for op in ops], [op.axis for op in ops], n
    )
    ctx.in_loop = False
    return pytree.tree_unflatten(list(res), out_spec)


def _sequential(body, n, operation):
    first = body(0)
    leaves, spec = pytree.tree_flatten(first)
    ops = _broadcast_ops(operation, first)
    state = [op.update(op.state(n, l), l, 0) for op, l in zip(ops, leaves)]
    for i in range(1, n):
        vals = pytree.tree_leaves(body(i))
        state = [op.update(s, v, i) for op, s, v in zip(ops, state, vals)]
    return pytree.tree_unflatten(state, spec)
