"""Graph rewrites applied to the captured step before it is clustered into tasks.

``fuse_norm_backward_adds``: in a pre-norm residual block the gradient of the block input is the sum of the
normalisation's input gradient and the gradient that arrives over the residual connection.  Autograd emits that as
``norm_bwd`` followed by an ``add`` kernel that re-reads both tensors; the fused op writes the sum in the pass that
produces the first operand.  The sum is rounded exactly as the two separate kernels would round it, so a rewritten
program still matches the eager step bit for bit.
"""
from __future__ import annotations

import operator

import torch
from torch import fx


def _val(n: fx.Node):
    return n.meta.get("val")


def fuse_norm_backward_adds(graph: fx.Graph) -> int:
    from ..ops import core as ops  # noqa: F401  (registers the ops)

    fused = {
        torch.ops.b200.rmsnorm_bwd.default: torch.ops.b200.rmsnorm_bwd_add.default,
        torch.ops.b200.layernorm_bwd.default: torch.ops.b200.layernorm_bwd_add.default,
    }
    order = {n: i for i, n in enumerate(graph.nodes)}
    count = 0
    for n in list(graph.nodes):
        if n.op != "call_function" or n.target not in fused:
            continue
        dx_items = [u for u in n.users if u.op == "call_function" and u.target is operator.getitem and u.args[1] == 0]
        if len(dx_items) != 1 or len(dx_items[0].users) != 1:
            continue
        dx = dx_items[0]
        add = next(iter(dx.users))
        if add.op != "call_function" or add.target is not torch.ops.aten.add.Tensor or add.kwargs or len(add.args) != 2:
            continue
        other = add.args[1] if add.args[0] is dx else add.args[0]
        if not isinstance(other, fx.Node) or other is dx or order[other] > order[n]:
            continue
        a, b = _val(dx), _val(other)
        if a is None or b is None or tuple(a.shape) != tuple(b.shape) or a.dtype != b.dtype:
            continue
        with graph.inserting_before(n):
            new = graph.call_function(fused[n.target], (*n.args, other))
        new.meta = dict(n.meta)
        n.replace_all_uses_with(new)
        add.replace_all_uses_with(dx)
        graph.erase_node(add)
        graph.erase_node(n)
        count += 1
    return count
