"""Marker ops that delimit pipeline stages and the microbatch loop in a captured train step.

These are the counterparts of the reference's IR primitives (src/jaxpp/jax_primitives.py):

=====================  ======================================================================
``pp::pipeline_yield``  stage boundary; identity on N tensors; its autograd formula emits a
                        backward-typed yield with the same stage id (reference :532-556)
``pp::loop_begin``      start of the microbatch loop: yields one slice of each batched input
``pp::loop_index``      the microbatch counter as a 0-d int64 tensor
``pp::loop_end``        end of the loop: per output an accumulation kind (Add / Concat / Max)
                        (together these three play the role of ``dax_pscan``, :559-614)
``pp::add_multi``       n-ary add of tensors living on different pipeline ranks (:57-108)
``pp::gather_multi``    stack of tensors living on different pipeline ranks (:189-255)
``pp::place_with``      identity placement hint (:526-530)
=====================  ======================================================================

They only ever execute on fake tensors while a step is being traced (the compiler removes or
lowers every one of them); their eager implementations exist so that un-jitted code still runs.
"""
from __future__ import annotations

import contextlib
import dataclasses
from typing import Any

import torch
from torch import Tensor


_lib = torch.library.Library("pp", "DEF")

FWD_CODE, BWD_CODE = 0, 1
OP_ADD, OP_CONCAT, OP_MAX = 0, 1, 2


def _clone_all(xs):
    return [x.clone() for x in xs]


# ---- pipeline_yield -------------------------------------------------------------------------
_lib.define("pipeline_yield(Tensor[] xs, int stage_id, int task_type, str name) -> Tensor[]")
_lib.impl("pipeline_yield", lambda xs, stage_id, task_type, name: _clone_all(xs), "CompositeExplicitAutograd")
torch.library.register_fake("pp::pipeline_yield", lambda xs, s, t, n: [torch.empty_like(x) for x in xs])


def _yield_setup(ctx, inputs, output):
    ctx.stage_id, ctx.name = inputs[1], inputs[3]


def _yield_bwd(ctx, grads):
    grads = list(grads)
    live = [i for i, g in enumerate(grads) if g is not None]
    outs = torch.ops.pp.pipeline_yield([grads[i].contiguous() for i in live], ctx.stage_id, BWD_CODE, ctx.name)
    full = [None] * len(grads)
    for i, o in zip(live, outs):
        full[i] = o
    return full, None, None, None


torch.library.register_autograd("pp::pipeline_yield", _yield_bwd, setup_context=_yield_setup)

# ---- loop markers ---------------------------------------------------------------------------
_lib.define("loop_begin(Tensor[] xs, int axis, int n) -> Tensor[]")
_lib.impl("loop_begin", lambda xs, axis, n: [x.select(axis, 0).clone() for x in xs], "CompositeExplicitAutograd")
torch.library.register_fake(
    "pp::loop_begin", lambda xs, axis, n: [x.new_empty([s for d, s in enumerate(x.shape) if d != axis % x.dim()]) for x in xs]
)

_lib.define("loop_index(int n, Device device) -> Tensor")
_lib.impl("loop_index", lambda n, device: torch.zeros((), dtype=torch.int64, device=device), "CompositeExplicitAutograd")
torch.library.register_fake("pp::loop_index", lambda n, device: torch.empty((), dtype=torch.int64, device=device))


def _loop_end_shapes(outs, kinds, axes, n):
    res = []
    for o, k, a in zip(outs, kinds, axes):
        if k == OP_CONCAT:
            shape = list(o.shape)
            shape.insert(a, n)
            res.append(o.new_empty(shape))
        else:
            res.append(torch.empty_like(o))
    return res


_lib.define("loop_end(Tensor[] outs, int[] kinds, int[] axes, int n) -> Tensor[]")
_lib.impl("loop_end", _loop_end_shapes, "CompositeExplicitAutograd")
torch.library.register_fake("pp::loop_end", _loop_end_shapes)

# ---- cross-rank collectives and hints -----------------------------------------------------------
_lib.define("add_multi(Tensor[] xs) -> Tensor")
_lib.impl("add_multi", lambda xs: torch.stack(list(xs)).sum(0) if len(xs) > 1 else xs[0].clone(), "CompositeExplicitAutograd")
torch.library.register_fake("pp::add_multi", lambda xs: torch.empty_like(xs[0]))

_lib.define("gather_multi(Tensor[] xs, int axis) -> Tensor")
_lib.impl("gather_multi", lambda xs, axis: torch.cat(list(xs), dim=axis), "CompositeExplicitAutograd")


def _gather_fake(xs, axis):
    shape = list(xs[0].shape)
    shape[axis] = sum(x.shape[axis] for x in xs)
    return xs[0].new_empty(shape)


torch.library.register_fake("pp::gather_multi", _gather_fake)

_lib.define("place_with(Tensor val, Tensor with_val) -> Tensor")
_lib.impl("place_with", lambda val, with_val: val.clone(), "CompositeExplicitAutograd")
torch.library.register_fake("pp::place_with", lambda val, with_val: torch.empty_like(val))
torch.library.register_autograd(
    "pp::place_with", lambda ctx, g: (g, None), setup_context=lambda ctx, inputs, output: None
)


# ---- trace context ---------------------------------------------------------------------------
@dataclasses.dataclass
class TraceContext:
    """State of one in-progress capture: the stage counter and what the loop looked like."""

    stage_counter: int = 0
    n_loops: int = 0
    schedule: Any = None
    n_mubatches: int | None = None
    in_loop: bool = False
    stage_names: dict = dataclasses.field(default_factory=dict)


_TRACE_STACK: list[TraceContext] = []


def current_trace() -> TraceContext | None:
    return _TRACE_STACK[-1] if _TRACE_STACK else None


@contextlib.contextmanager
def yield_scope():
    """Activate stage markers; resets the stage counter (reference: pipelining.py:25-36)."""
    ctx = TraceContext()
    _TRACE_STACK.append(ctx)
    try:
        yield ctx
    finally:
        _TRACE_STACK.pop()


MARKER_TARGETS = None


def marker_targets():
    global MARKER_TARGETS
    if MARKER_TARGETS is None:
        MARKER_TARGETS = {
            "yield": torch.ops.pp.pipeline_yield.default,
            "loop_begin": torch.ops.pp.loop_begin.default,
            "loop_index": torch.ops.pp.loop_index.default,
            "loop_end": torch.ops.pp.loop_end.default,
            "add_multi": torch.ops.pp.add_multi.default,
            "gather_multi": torch.ops.pp.gather_multi.default,
            "place_with": torch.ops.pp.place_with.default,
        }
    return MARKER_TARGETS
