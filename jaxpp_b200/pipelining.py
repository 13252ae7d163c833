"""Stage markers (reference: src/jaxpp/pipelining.py:39-81)."""
from __future__ import annotations

import warnings
from typing import Any

import torch
from torch.utils import _pytree as pytree

from .primitives import FWD_CODE, current_trace, yield_scope

__all__ = ["mark_stage_end", "pipeline_enter_stage", "yield_scope"]


def mark_stage_end(anchor: Any, name: str | None = None) -> Any:
    """Mark everything computed so far (since the previous marker) as one pipeline stage.

    ``anchor`` is a pytree of tensors that flow into the next stage; it is returned unchanged in
    value.  A marker is also required after the *last* stage.  Outside a captured step (plain
    eager execution, i.e. the un-pipelined oracle) this is a no-op.
    """
    ctx = current_trace()
    if ctx is None:
        return anchor
    leaves, spec = pytree.tree_flatten(anchor)
    tensor_pos = [i for i, l in enumerate(leaves) if isinstance(l, torch.Tensor)]
    if not tensor_pos:
        return anchor
    stage_id = ctx.stage_counter
    ctx.stage_counter += 1
    if name is not None:
        ctx.stage_names[stage_id] = name
    outs = torch.ops.pp.pipeline_yield([leaves[i] for i in tensor_pos], stage_id, FWD_CODE, name or "")
    for i, o in zip(tensor_pos, outs):
        leaves[i] = o
    return pytree.tree_unflatten(leaves, spec)


def pipeline_enter_stage(anchor: Any, name: str | None = None) -> Any:
    """Deprecated spelling of :func:`mark_stage_end` (the reference keeps it with a warning)."""
    warnings.warn("pipeline_enter_stage is deprecated, use mark_stage_end", DeprecationWarning, stacklevel=2)
    return mark_stage_end(anchor, name)
