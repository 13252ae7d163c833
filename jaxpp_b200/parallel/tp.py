"""Tensor-parallel (Megatron sequence-parallel) building blocks inside one pipeline stage.

The reference leaves intra-stage parallelism to XLA's SPMD partitioner (src/jaxpp/core.py:2970-3024);
here it is explicit.  Activations between blocks are sharded over tokens along the ``model`` mesh axis:

* ``column_linear``: ``y = all_gather(x) @ W_shard^T``      — op ``b200::ag_linear``  (all-gather → GEMM)
* ``row_linear``   : ``y = reduce_scatter(x @ W_shard^T)``  — op ``b200::linear_rs``  (GEMM → reduce-scatter)

Each op has two implementations chosen by ``JAXPP_B200_FUSED_COLLECTIVES``: the fused sm_100a kernels
that move tiles over NVLink peer memory from inside the GEMM (``jaxpp_b200.parallel.fused``), and the
plain NCCL collective followed/preceded by the GEMM (the measured baseline).  Their backward passes are
again fused ops (the transpose of all-gather→GEMM is GEMM→reduce-scatter and vice versa), with dgrad
and wgrad kept separate for zero-bubble schedules.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ..mesh import MpmdMesh
from ..ops import core as ops
from ..utils import config

_lib = torch.library.Library("b200tp", "DEF")


# ---- mesh helpers ----------------------------------------------------------------------------------------
def axis_size(axis: str) -> int:
    return MpmdMesh.current().shape[axis]


def axis_rank(axis: str) -> int:
    mesh = MpmdMesh.current()
    if mesh.shape[axis] == 1:
        return 0
    return mesh.axis_index(axis)


def _group(axis: str):
    return MpmdMesh.current().axis_group(axis)


def _fused(t: Tensor) -> bool:
    return t.is_cuda and config.use_fused_collectives.value and config.use_native_kernels.value


# ---- raw collectives (NCCL / gloo) ----------------------------------------------------------------------------
def _all_gather_rows(x: Tensor, axis: str) -> Tensor:
    n = axis_size(axis)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((n * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=_group(axis))
    return out


def _reduce_scatter_rows(x: Tensor, axis: str) -> Tensor:
    n = axis_size(axis)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] // n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x, group=_group(axis))
    else:  # gloo has no reduce_scatter
        tmp = x.clone()
        dist.all_reduce(tmp, group=_group(axis))
        r = axis_rank(axis)
        out.copy_(tmp[r * out.shape[0]:(r + 1) * out.shape[0]])
    return out


def _all_reduce_impl(x: Tensor, axis: str) -> Tensor:
    if axis_size(axis) == 1:
        return x
    if _fused(x) and x.dtype in (torch.float32, torch.bfloat16):
        from . import fused

        if x.numel() * x.element_size() >= fused.AR_MIN_BYTES:
            return fused.all_reduce(x, axis)
    out = x.contiguous().clone()
    dist.all_reduce(out, group=_group(axis))
    return out


def _rows_fake(x, axis, mult=None, div=None):
    n = axis_size(axis)
    rows = x.shape[0] * n if mult else x.shape[0] // n
    return x.new_empty((rows, *x.shape[1:]))


_lib.define("all_gather(Tensor x, str axis) -> Tensor")
_lib.impl("all_gather", _all_gather_rows, "CompositeExplicitAutograd")
torch.library.register_fake("b200tp::all_gather", lambda x, axis: _rows_fake(x, axis, mult=True))

_lib.define("reduce_scatter(Tensor x, str axis) -> Tensor")
_lib.impl("reduce_scatter", _reduce_scatter_rows, "CompositeExplicitAutograd")
torch.library.register_fake("b200tp::reduce_scatter", lambda x, axis: _rows_fake(x, axis, div=True))

_lib.define("all_reduce(Tensor x, str axis) -> Tensor")
_lib.impl("all_reduce", _all_reduce_impl, "CompositeExplicitAutograd")
torch.library.register_fake("b200tp::all_reduce", lambda x, axis: torch.empty_like(x))

torch.library.register_autograd(
    "b200tp::all_gather",
    lambda ctx, g: (torch.ops.b200tp.reduce_scatter(g.contiguous(), ctx.axis), None),
    setup_context=lambda ctx, inputs, output: setattr(ctx, "axis", inputs[1]),
)
torch.library.register_autograd(
    "b200tp::reduce_scatter",
    lambda ctx, g: (torch.ops.b200tp.all_gather(g.contiguous(), ctx.axis), None),
    setup_context=lambda ctx, inputs, output: setattr(ctx, "axis", inputs[1]),
)


def all_reduce(x: Tensor, axis: str) -> Tensor:
    return torch.ops.b200tp.all_reduce(x, axis)


# ---- fused ops -------------------------------------------------------------------------------------------------
def _ag_linear_impl(x, w, bias, axis):
    if _fused(x) and axis_size(axis) > 1:
        from . import fused

        return fused.ag_linear(x, w, bias, axis)
    return ops.linear(_all_gather_rows(x, axis), w, bias)


def _linear_rs_impl(x, w, axis):
    if _fused(x) and axis_size(axis) > 1:
        from . import fused

        return fused.linear_rs(x, w, axis)
    return _reduce_scatter_rows(ops.linear(x, w, None), axis)


def _dgrad_rs_impl(dy, w, axis):
    """dx_shard = reduce_scatter(dy @ W)"""
    if _fused(dy) and axis_size(axis) > 1:
        from . import fused

        return fused.dgrad_rs(dy, w, axis)
    return _reduce_scatter_rows(ops.linear_dgrad(dy, w), axis)


def _ag_wgrad_impl(dy, x_shard, axis, out_dtype=None):
    """dW = dy^T @ all_gather(x_shard)"""
    if _fused(dy) and axis_size(axis) > 1:
        from . import fused

        return fused.ag_wgrad(dy, x_shard, axis, out_dtype)
    return ops.linear_wgrad(dy, _all_gather_rows(x_shard, axis), out_dtype)


def _ag_dgrad_impl(dy_shard, w, axis):
    """(dx, dy_full) with dy_full = all_gather(dy_shard), dx = dy_full @ W"""
    if _fused(dy_shard) and axis_size(axis) > 1:
        from . import fused

        return fused.ag_dgrad(dy_shard, w, axis)
    full = _all_gather_rows(dy_shard, axis)
    return ops.linear_dgrad(full, w), full


_lib.define("ag_linear(Tensor x, Tensor w, Tensor? bias, str axis) -> Tensor")
_lib.impl("ag_linear", _ag_linear_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200tp::ag_linear", lambda x, w, bias, axis: x.new_empty(x.shape[0] * axis_size(axis), w.shape[0])
)
_lib.define("linear_rs(Tensor x, Tensor w, str axis) -> Tensor")
_lib.impl("linear_rs", _linear_rs_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200tp::linear_rs", lambda x, w, axis: x.new_empty(x.shape[0] // axis_size(axis), w.shape[0])
)
_lib.define("dgrad_rs(Tensor dy, Tensor w, str axis) -> Tensor")
_lib.impl("dgrad_rs", _dgrad_rs_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200tp::dgrad_rs", lambda dy, w, axis: dy.new_empty(dy.shape[0] // axis_size(axis), w.shape[1])
)
_lib.define("ag_wgrad(Tensor dy, Tensor x_shard, str axis, ScalarType? out_dtype=None) -> Tensor")
_lib.impl("ag_wgrad", _ag_wgrad_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200tp::ag_wgrad", lambda dy, x, axis, out_dtype=None: dy.new_empty(dy.shape[1], x.shape[1], dtype=out_dtype or dy.dtype)
)
_lib.define("ag_dgrad(Tensor dy_shard, Tensor w, str axis) -> (Tensor, Tensor)")
_lib.impl("ag_dgrad", _ag_dgrad_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200tp::ag_dgrad",
    lambda dy, w, axis: (dy.new_empty(dy.shape[0] * axis_size(axis), w.shape[1]),
                         dy.new_empty(dy.shape[0] * axis_size(axis), dy.shape[1])),
)


for _name, _fn in (("all_gather", _all_gather_rows), ("reduce_scatter", _reduce_scatter_rows), ("all_reduce", _all_reduce_impl),
                   ("ag_linear", _ag_linear_impl), ("linear_rs", _linear_rs_impl), ("dgrad_rs", _dgrad_rs_impl),
                   ("ag_wgrad", _ag_wgrad_impl), ("ag_dgrad", _ag_dgrad_impl)):
    ops.DIRECT[getattr(torch.ops.b200tp, _name).default] = _fn      # see ops.core.DIRECT


def _ag_linear_setup(ctx, inputs, output):
    x, w, bias, axis = inputs
    ctx.save_for_backward(x, w)
    ctx.axis, ctx.has_bias = axis, bias is not None


def _ag_linear_bwd(ctx, dy):
    x, w = ctx.saved_tensors
    dy = dy.contiguous()
    dx = torch.ops.b200tp.dgrad_rs(dy, w, ctx.axis) if ctx.needs_input_grad[0] else None
    dw = torch.ops.b200tp.ag_wgrad(dy, x, ctx.axis, ops.WGRAD_DTYPE[0]) if ctx.needs_input_grad[1] else None
    db = ops.colsum(dy) if ctx.has_bias and ctx.needs_input_grad[2] else None
    return dx, dw, db, None


torch.library.register_autograd("b200tp::ag_linear", _ag_linear_bwd, setup_context=_ag_linear_setup)


def _linear_rs_setup(ctx, inputs, output):
    x, w, axis = inputs
    ctx.save_for_backward(x, w)
    ctx.axis = axis


def _linear_rs_bwd(ctx, dy_shard):
    x, w = ctx.saved_tensors
    dx, dy_full = torch.ops.b200tp.ag_dgrad(dy_shard.contiguous(), w, ctx.axis)
    dw = ops.linear_wgrad(dy_full, x, ops.WGRAD_DTYPE[0]) if ctx.needs_input_grad[1] else None
    return (dx if ctx.needs_input_grad[0] else None), dw, None


torch.library.register_autograd("b200tp::linear_rs", _linear_rs_bwd, setup_context=_linear_rs_setup)


# ---- model-facing helpers --------------------------------------------------------------------------------------
def column_linear(x: Tensor, w: Tensor, bias, cfg) -> Tensor:
    """Column-parallel linear on token-sharded input: gathers tokens, output features are sharded."""
    if cfg.tp == 1:
        return ops.linear(x, w, bias)
    return torch.ops.b200tp.ag_linear(x, w, bias, cfg.tp_axis)


def row_linear(x: Tensor, w: Tensor, bias, cfg) -> Tensor:
    """Row-parallel linear: input features are sharded, output is summed over the axis and token-sharded.
    The bias is added once, after the reduction."""
    if cfg.tp == 1:
        return ops.linear(x, w, bias)
    y = torch.ops.b200tp.linear_rs(x, w, cfg.tp_axis)
    return y if bias is None else y + bias


def local_token_slice(flat: Tensor, cfg) -> Tensor:
    """This device's contiguous slice of the flattened (batch-major) token dimension."""
    n = flat.shape[0] // cfg.tp
    r = axis_rank(cfg.tp_axis)
    return flat[r * n:(r + 1) * n]


def local_positions(n_local: int, cfg, device) -> Tensor:
    """Position ids of this device's token slice."""
    r = axis_rank(cfg.tp_axis) if cfg.tp > 1 else 0
    start = r * n_local
    return (torch.arange(n_local, device=device) + start) % cfg.seq


# ---- vocabulary-parallel cross entropy ---------------------------------------------------------------------------
def _vp_ce_impl(logits: Tensor, labels: Tensor, axis: str):
    """logits [T, V/n] (this rank's slice of the vocabulary, rank r holds entries [r V/n, (r+1) V/n)), labels [T] ->
    (loss [T] fp32, lse [T] fp32), both the same on every rank of ``axis``."""
    n = axis_size(axis)
    lf = logits.float()
    local_lse = torch.logsumexp(lf, dim=-1)
    if n == 1:
        return local_lse - lf.gather(1, labels.view(-1, 1)).view(-1), local_lse
    r = axis_rank(axis)
    width = logits.shape[-1]
    every = torch.empty(n * local_lse.shape[0], dtype=torch.float32, device=logits.device)
    dist.all_gather_into_tensor(every, local_lse.contiguous(), group=_group(axis))
    lse = torch.logsumexp(every.view(n, -1), dim=0)                       # stable: combines the ranks' log-sum-exps
    local = labels - r * width
    mine = (local >= 0) & (local < width)
    target = lf.gather(1, local.clamp(0, width - 1).view(-1, 1)).view(-1) * mine
    dist.all_reduce(target, group=_group(axis))                           # the owner of the label's entry contributes
    return lse - target, lse


def _vp_ce_bwd_impl(dloss: Tensor, logits: Tensor, labels: Tensor, lse: Tensor, axis: str) -> Tensor:
    """The loss is one value per token shared by the ranks: the gradients the ranks hold for it add up, then every
    rank forms its slice of softmax - onehot."""
    n = axis_size(axis)
    dl = dloss.float().contiguous().clone()
    r = 0
    if n > 1:
        dist.all_reduce(dl, group=_group(axis))
        r = axis_rank(axis)
    width = logits.shape[-1]
    p = torch.exp(logits.float() - lse.unsqueeze(-1))
    local = labels - r * width
    mine = (local >= 0) & (local < width)
    p.scatter_add_(1, local.clamp(0, width - 1).view(-1, 1), -mine.to(p.dtype).view(-1, 1))
    return (p * dl.unsqueeze(-1)).to(logits.dtype)


_lib.define("vocab_parallel_ce(Tensor logits, Tensor labels, str axis) -> (Tensor, Tensor)")
_lib.impl("vocab_parallel_ce", _vp_ce_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200tp::vocab_parallel_ce",
    lambda logits, labels, axis: (logits.new_empty(logits.shape[0], dtype=torch.float32),
                                  logits.new_empty(logits.shape[0], dtype=torch.float32)))
_lib.define("vocab_parallel_ce_bwd(Tensor dloss, Tensor logits, Tensor labels, Tensor lse, str axis) -> Tensor")
_lib.impl("vocab_parallel_ce_bwd", _vp_ce_bwd_impl, "CompositeExplicitAutograd")
torch.library.register_fake("b200tp::vocab_parallel_ce_bwd", lambda dloss, logits, labels, lse, axis: torch.empty_like(logits))


ops.DIRECT[torch.ops.b200tp.vocab_parallel_ce.default] = _vp_ce_impl
ops.DIRECT[torch.ops.b200tp.vocab_parallel_ce_bwd.default] = _vp_ce_bwd_impl


def _vp_ce_setup(ctx, inputs, output):
    logits, labels, axis = inputs
    ctx.save_for_backward(logits, labels, output[1])
    ctx.axis = axis


def _vp_ce_backward(ctx, dloss, dlse):
    logits, labels, lse = ctx.saved_tensors
    return torch.ops.b200tp.vocab_parallel_ce_bwd(dloss.contiguous(), logits, labels, lse, ctx.axis), None, None


torch.library.register_autograd("b200tp::vocab_parallel_ce", _vp_ce_backward, setup_context=_vp_ce_setup)


def vocab_parallel_cross_entropy(logits: Tensor, labels: Tensor, axis: str) -> Tensor:
    """Per-token cross entropy from logits whose vocabulary dimension is split over ``axis`` (the full [tokens, vocab]
    matrix is never assembled): log-sum-exps are combined across the ranks, the label's logit comes from its owner."""
    return torch.ops.b200tp.vocab_parallel_ce(logits, labels, axis)[0]
