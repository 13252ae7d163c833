"""Optimizer state sharded over the data-parallel ranks (ZeRO stage 1).

Every data-parallel rank keeps the fp32 master copy and the Adam moments of a 1/n slice of each (flattened,
zero-padded) parameter.  After the microbatch loop the gradient is reduce-scattered instead of all-reduced, the
fused AdamW kernel updates the slice and emits its bf16 copy, and the low-precision parameter is all-gathered
from the owners of the slices:

    g_shard = reduce_scatter_flat(g)             # [S]   S = shard_numel(numel, n)
    master', m', v', lp = adamw(master, g_shard, m, v, ...)
    p'      = all_gather_flat(lp, numel).view(shape)

The slices are padded per axis size, so a checkpoint of sliced optimizer state restores into the same data-parallel
size only (the parameters themselves restore into any layout).

On GPUs both collectives are one peer-memory kernel each (the two halves of the one-kernel all-reduce,
``csrc/collectives.cu``); elsewhere, and below 1 MiB, NCCL / gloo.  The reference leaves this to XLA's SPMD
partitioner: a parameter annotated ``P("fsdp")`` gets a cast + all-gather before the loop and a reduce-scatter
after it (PERF_GUIDE.md:27-70, examples/tutorial.ipynb cell 7).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from . import tp as tpmod

_lib = torch.library.Library("b200dp", "DEF")

FUSED_MIN_BYTES = 1 << 20   # smaller tensors are latency-bound: leave them to the library collective


def shard_numel(numel: int, n: int) -> int:
    """Elements per rank of a flat tensor of ``numel`` elements split over ``n`` ranks: padded so that a slice is a
    whole number of 16-byte vectors for 2- and 4-byte element types alike."""
    return (numel + 8 * n - 1) // (8 * n) * 8


def local_shard(t: Tensor, n: int, r: int) -> Tensor:
    """Slice ``r`` of ``n`` of the flattened, zero-padded ``t`` (a copy)."""
    s = shard_numel(t.numel(), n)
    flat = t.detach().reshape(-1)
    out = flat.new_zeros(s)
    lo, hi = r * s, min((r + 1) * s, flat.numel())
    if hi > lo:
        out[:hi - lo] = flat[lo:hi]
    return out


def _use_fused(x: Tensor, nbytes: int) -> bool:
    return tpmod._fused(x) and x.dtype in (torch.float32, torch.bfloat16) and nbytes >= FUSED_MIN_BYTES


def _reduce_scatter_impl(x: Tensor, axis: str, scale: float) -> Tensor:
    n = tpmod.axis_size(axis)
    s = shard_numel(x.numel(), n)
    if n == 1:
        out = local_shard(x, 1, 0)
        return out if scale == 1.0 else out * scale
    if _use_fused(x, x.numel() * x.element_size()):
        from . import fused

        return fused.reduce_scatter_flat(x, axis, scale)
    flat = x.contiguous().view(-1)
    padded = flat.new_zeros(s * n)
    padded[:flat.numel()] = flat
    r = tpmod.axis_rank(axis)
    if x.is_cuda:
        out = flat.new_empty(s)
        dist.reduce_scatter_tensor(out, padded, group=tpmod._group(axis))
    else:  # gloo has no reduce_scatter
        dist.all_reduce(padded, group=tpmod._group(axis))
        out = padded[r * s:(r + 1) * s].clone()
    return out if scale == 1.0 else out * scale


def _all_gather_impl(shard: Tensor, axis: str, numel: int) -> Tensor:
    n = tpmod.axis_size(axis)
    shard = shard.contiguous().view(-1)
    if n == 1:
        return shard[:numel].clone()
    if _use_fused(shard, shard.numel() * shard.element_size() * n):
        from . import fused

        return fused.all_gather_flat(shard, axis)[:numel]
    out = shard.new_empty(shard.numel() * n)
    dist.all_gather_into_tensor(out, shard, group=tpmod._group(axis))
    return out[:numel]


_lib.define("reduce_scatter_flat(Tensor x, str axis, float scale) -> Tensor")
_lib.impl("reduce_scatter_flat", _reduce_scatter_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200dp::reduce_scatter_flat", lambda x, axis, scale: x.new_empty((shard_numel(x.numel(), tpmod.axis_size(axis)),)))

_lib.define("all_gather_flat(Tensor shard, str axis, int numel) -> Tensor")
_lib.impl("all_gather_flat", _all_gather_impl, "CompositeExplicitAutograd")
torch.library.register_fake("b200dp::all_gather_flat", lambda shard, axis, numel: shard.new_empty((numel,)))


def reduce_scatter_flat(x: Tensor, axis: str, scale: float = 1.0) -> Tensor:
    """This rank's slice of scale * (sum of ``x`` over the ranks of ``axis``), flattened and zero-padded."""
    return torch.ops.b200dp.reduce_scatter_flat(x, axis, float(scale))


def all_gather_flat(shard: Tensor, axis: str, numel: int) -> Tensor:
    """The first ``numel`` elements of the concatenation of every rank's ``shard``."""
    return torch.ops.b200dp.all_gather_flat(shard, axis, int(numel))


def shard_optimizer_state(state: dict, n: int, r: int, keep=lambda path: False) -> dict:
    """Turn a training state with full-size ``master`` / ``m`` / ``v`` trees into one whose leaves are rank ``r``'s
    slices; leaves that are not tensors (placeholders of other pipeline ranks) become placeholders of the slice
    shape, and leaves for which ``keep(path)`` is true (parameters that are not replicated over the axis, such as
    experts sharded over it) stay whole."""
    from ..core import ShapeDtypeStruct

    def walk(tree, path=()):
        if isinstance(tree, dict):
            return {k: walk(v, path + (k,)) for k, v in tree.items()}
        if keep(path):
            return tree
        if isinstance(tree, ShapeDtypeStruct):
            numel = 1
            for d in tree.shape:
                numel *= int(d)
            return ShapeDtypeStruct((shard_numel(numel, n),), tree.dtype)
        return local_shard(tree, n, r)

    out = dict(state)
    for key in ("master", "m", "v"):
        out[key] = walk(state[key])
    return out

def _register_direct_calls():
    """Generated task code calls these implementations without the dispatcher (see ops.core.DIRECT)."""
    from ..ops import core as _core

    _core.DIRECT[torch.ops.b200dp.reduce_scatter_flat.default] = _reduce_scatter_impl
    _core.DIRECT[torch.ops.b200dp.all_gather_flat.default] = _all_gather_impl


_register_direct_calls()
