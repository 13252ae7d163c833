"""Capture of a user train step as one flat dataflow graph.

The step function is traced once with ``make_fx`` on CPU *fake* tensors (no data, no GPU), so
that the result is a ``torch.fx`` graph whose nodes are the ``b200::*`` custom ops, ATen glue,
and the ``pp::*`` markers.  Because ``torch.autograd.grad`` runs *inside* the traced function,
the graph already contains forward and backward — the same shape of IR the reference obtains by
tracing ``jax.grad`` to a jaxpr (src/jaxpp/core.py:3173-3259).  Device constants recorded in the
graph are re-bound to the executing device when tasks are generated, so a program captured on a
CPU-only machine runs unchanged on a GPU.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Sequence

import torch
from torch import fx
from torch.fx.experimental.proxy_tensor import make_fx
from torch.utils import _pytree as pytree

from .. import primitives as prim
from ..training import _TRACE_DEVICE
from ..utils import log_elapsed_time


@dataclasses.dataclass(frozen=True)
class ArgMeta:
    """Shape/dtype of one flat tensor argument (the local shard seen by one device)."""

    shape: tuple[int, ...]
    dtype: torch.dtype

    @staticmethod
    def of(x) -> "ArgMeta":
        return ArgMeta(tuple(x.shape), x.dtype)


@dataclasses.dataclass
class Captured:
    gm: fx.GraphModule
    graph: fx.Graph
    placeholders: list[fx.Node]  # one per flat tensor input, in order
    outputs: list[Any]  # flat outputs: fx.Node or a Python constant
    out_spec: Any
    trace: prim.TraceContext


def value_meta(node: fx.Node):
    """The fake tensor (or nested structure of them) recorded for ``node``."""
    return node.meta.get("val")


def capture(fn: Callable, in_spec, tensor_metas: Sequence[ArgMeta], static_leaves: dict[int, Any],
            n_leaves: int) -> Captured:
    """Trace ``fn(*args, **kwargs)`` where the flattened inputs are described by ``tensor_metas``
    (tensor leaves, in flat order) and ``static_leaves`` (flat position → Python value)."""
    tensor_positions = [i for i in range(n_leaves) if i not in static_leaves]
    assert len(tensor_positions) == len(tensor_metas)

    out_box: dict[str, Any] = {}

    def flat_fn(*tensors):
        leaves: list[Any] = [None] * n_leaves
        for pos, t in zip(tensor_positions, tensors):
            leaves[pos] = t
        for pos, v in static_leaves.items():
            leaves[pos] = v
        args, kwargs = pytree.tree_unflatten(leaves, in_spec)
        out = fn(*args, **kwargs)
        out_leaves, out_spec = pytree.tree_flatten(out)
        out_box["spec"] = out_spec
        tensor_out = []
        kinds = []
        for o in out_leaves:
            if isinstance(o, torch.Tensor):
                kinds.append(("t", len(tensor_out)))
                tensor_out.append(o)
            else:
                kinds.append(("c", o))
        out_box["kinds"] = kinds
        return tensor_out

    from torch._subclasses.fake_tensor import FakeTensorMode

    fake_mode = FakeTensorMode(allow_non_fake_inputs=True)
    with fake_mode:
        fakes = [torch.empty(m.shape, dtype=m.dtype, device="cpu") for m in tensor_metas]
    with log_elapsed_time("capture/tracing"), prim.yield_scope() as ctx:
        _TRACE_DEVICE.append(torch.device("cpu"))
        try:
            gm = make_fx(flat_fn, tracing_mode="fake", _allow_non_fake_inputs=True)(*fakes)
        finally:
            _TRACE_DEVICE.pop()
    graph = gm.graph
    placeholders = [n for n in graph.nodes if n.op == "placeholder"]
    out_node = next(n for n in graph.nodes if n.op == "output")
    traced_outs = out_node.args[0]
    outputs = []
    for kind, payload in out_box["kinds"]:
        outputs.append(traced_outs[payload] if kind == "t" else payload)
    return Captured(gm, graph, placeholders, outputs, out_box["spec"], ctx)
