"""Weight-gradient sinks: let a wgrad GEMM add into the loop's accumulator instead of producing a fresh tensor.

A ``treduce`` loop sums every microbatch's weight gradient into an accumulator.  Done literally that is a GEMM
that writes a parameter-sized fp32 tensor followed by an add kernel that reads two of them and writes one, per
weight and microbatch.  When a task output is (a) produced by a weight-gradient op and (b) consumed by nothing but
the loop's ``Add`` accumulation, the executor hands the accumulator to the task and the op's GEMM epilogue does
``acc += dy^T x`` in place (the accumulate epilogue of the tcgen05 kernels; ``add_`` on the reference path) and
returns the accumulator itself, which makes the accumulation step a no-op.  The reference reaches the same effect
through XLA's fusion of the add into the loop body; this is the explicit form of row N16 of the design inventory.
"""
from __future__ import annotations

import torch

from . import core as ops


def sink_targets() -> tuple:
    """Op overloads whose result may be redirected into an accumulator."""
    out = [torch.ops.b200.linear_wgrad.default, torch.ops.b200.embedding_bwd.default, torch.ops.b200.linear_wgrad_batched.default]
    try:
        from ..parallel import tp  # noqa: F401  (registers the b200tp ops)

        out.append(torch.ops.b200tp.ag_wgrad.default)
    except Exception:  # pragma: no cover - the tensor-parallel ops are always importable
        pass
    return tuple(out)


def early_collective_targets() -> tuple:
    """Collectives on a summed gradient that may be issued from inside the task that completes the sum."""
    from ..parallel import tp, zero  # noqa: F401  (register the ops)

    return (torch.ops.b200tp.all_reduce.default, torch.ops.b200dp.reduce_scatter_flat.default)


def _fits(acc: torch.Tensor, rows: int, cols: int, out_dtype) -> bool:
    return acc.dim() == 2 and acc.shape[0] == rows and acc.shape[1] == cols and (out_dtype is None or acc.dtype == out_dtype)


def accumulate(op, acc: torch.Tensor, *args, **kwargs) -> torch.Tensor:
    """``acc += op(*args)`` with the addition done by the op where it can; returns ``acc``."""
    if op is torch.ops.b200.linear_wgrad.default:
        dy, x = args[0], args[1]
        out_dtype = args[2] if len(args) > 2 else kwargs.get("out_dtype")
        if (ops._use_native(dy) and acc.dtype == torch.float32 and acc.is_contiguous()
                and _fits(acc, dy.shape[-1], x.shape[-1], out_dtype) and dy.dtype == torch.bfloat16):
            ops._native().linear_wgrad(dy, x, out=acc, accumulate=True)
            return acc
    elif op is torch.ops.b200.embedding_bwd.default:
        dy, ids, vocab = args[0], args[1], args[2]
        if (ops._use_native(dy) and acc.dtype == torch.float32 and acc.is_contiguous() and acc.dim() == 2
                and acc.shape[0] == vocab and acc.shape[1] == dy.shape[-1]):
            ops._native().embedding_bwd(dy, ids, vocab, out=acc, accumulate=True)   # scatter-add into the accumulator
            return acc
    elif op is torch.ops.b200.linear_wgrad_batched.default:
        # expert weight gradients: [E, N, K] per microbatch is the largest tensor a mixture-of-experts backward produces
        dy, x = args[0], args[1]
        counts = args[3] if len(args) > 3 else kwargs.get("counts")
        seg_rows = args[4] if len(args) > 4 else kwargs.get("seg_rows", 0)
        if (ops._use_native(dy) and acc.dtype == torch.float32 and acc.is_contiguous() and dy.dtype == torch.bfloat16
                and acc.dim() == 3 and tuple(acc.shape) == (dy.shape[0], dy.shape[2], x.shape[2])):
            if ops._native().linear_wgrad_batched(dy, x, None, counts, seg_rows, out=acc, accumulate=True) is not None:
                return acc
    elif op is torch.ops.b200tp.ag_wgrad.default:
        dy, x_shard, axis = args[0], args[1], args[2]
        out_dtype = args[3] if len(args) > 3 else kwargs.get("out_dtype")
        from ..parallel import tp

        if (tp._fused(dy) and tp.axis_size(axis) > 1 and acc.dtype == torch.float32 and acc.is_contiguous()
                and _fits(acc, dy.shape[-1], x_shard.shape[-1], out_dtype)):
            from ..parallel import fused

            got = fused.ag_wgrad(dy, x_shard, axis, out_dtype, acc=acc)
            if got is acc:
                return acc
            return acc.add_(got)
        if (ops._use_native(dy) and acc.dtype == torch.float32 and acc.is_contiguous() and dy.dtype == torch.bfloat16
                and _fits(acc, dy.shape[-1], x_shard.shape[-1], out_dtype)):
            ops._native().linear_wgrad(dy, tp._all_gather_rows(x_shard, axis), out=acc, accumulate=True)
            return acc
    return acc.add_(op(*args, **kwargs))


class _Named:
    def __init__(self, fn, name):
        self.fn, self.__name__ = fn, name

    def __call__(self, *a, **k):
        return self.fn(*a, **k)

    def __str__(self):
        return self.__name__


def call(op, sink, index: int, *args, **kwargs):
    """What generated task code calls for a sinkable op: ``sink`` maps output positions to accumulators."""
    acc = sink.get(index) if sink else None
    if acc is None:
        return op(*args, **kwargs)
    from ..utils import optimes

    if isinstance(op, optimes.Timed):      # per-op timing is on: time the accumulating form under the op's name
        inner, s2 = op.target, {index: acc}
        return optimes.Timed(_Named(lambda *a, **k: call(inner, s2, index, *a, **k), op.name))(*args, **kwargs)
    if isinstance(acc, tuple):   # (accumulator, hook): the gradient is final after this contribution
        acc, hook = acc
        out = accumulate(op, acc, *args, **kwargs)
        hook(out)
        return out
    return accumulate(op, acc, *args, **kwargs)
