"""Public API (reference: src/jaxpp/api.py:19-65)."""
from __future__ import annotations

from typing import Sequence

import torch

from .array import (DistArray, MpmdArray, MpmdSharding, _to_global_array, mpmd_to_spmd_reshard, reshard,
                    spmd_to_mpmd_reshard)
from .core import (CompiledMpmd, MpmdFunction, ShapeDtypeStruct, mpmd_jit_by_yield, mpmd_jit_with_loop,
                   value_and_grad)
from .mesh import Device, Mesh, MpmdMesh, NamedSharding, P, PartitionSpec
from .pipelining import mark_stage_end, pipeline_enter_stage
from .primitives import current_trace
from .runtime.executor import collect_task_times_ms
from .schedules import (BaseSchedule, DualPipeV, Eager1F1B, GPipe, Interleaved1F1B, InterleavedGPipe, KimiK2, Std1F1B,
                        ZeroBubble)
from .training import Add, Concat, Max, take, treduce, treduce_i

_to_global_jax_array = _to_global_array  # name under which the reference exports it


def cross_mpmd_all_reduce(*args: torch.Tensor) -> torch.Tensor:
    """Sum tensors that live on different pipeline ranks; the result lives on all of them.
    All arguments must have the same dtype (reference: api.py:48-54)."""
    if len(args) == 0:
        raise ValueError("cross_mpmd_all_reduce needs at least one argument")
    dtypes = {a.dtype for a in args}
    if len(dtypes) != 1:
        raise AssertionError(f"cross_mpmd_all_reduce arguments must share one dtype, got {sorted(map(str, dtypes))}")
    if current_trace() is None:
        out = args[0].clone()
        for a in args[1:]:
            out = out + a
        return out
    return torch.ops.pp.add_multi(list(args))


def cross_mpmd_stack(arrays: Sequence[torch.Tensor], axis: int = 0) -> torch.Tensor:
    """Stack tensors that live on different pipeline ranks along a new ``axis`` (reference: api.py:57-61)."""
    expanded = [a.unsqueeze(axis) for a in arrays]
    if current_trace() is None:
        return torch.cat(expanded, dim=axis)
    return torch.ops.pp.gather_multi(expanded, axis)


def place_with(val: torch.Tensor, with_val: torch.Tensor) -> torch.Tensor:
    """Hint: compute ``val`` on the pipeline rank (and in the task) where ``with_val`` lives."""
    if current_trace() is None:
        return val
    return torch.ops.pp.place_with(val, with_val)


__all__ = [
    "mpmd_jit_with_loop", "mpmd_jit_by_yield", "treduce", "treduce_i", "Add", "Max", "Concat", "mark_stage_end",
    "pipeline_enter_stage", "MpmdMesh", "MpmdArray", "MpmdSharding", "BaseSchedule", "Std1F1B", "Eager1F1B",
    "Interleaved1F1B", "KimiK2", "ZeroBubble", "DualPipeV", "GPipe", "cross_mpmd_all_reduce", "cross_mpmd_stack",
    "place_with", "spmd_to_mpmd_reshard", "mpmd_to_spmd_reshard", "collect_task_times_ms", "_to_global_jax_array",
    "value_and_grad", "take", "Mesh", "Device", "NamedSharding", "PartitionSpec", "P", "DistArray", "ShapeDtypeStruct",
]
