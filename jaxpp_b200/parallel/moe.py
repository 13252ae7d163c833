"""Mixture-of-experts building blocks with expert parallelism (Mixtral-style top-k routing).

The reference has no MoE support (only an ``"expert"`` axis name in a mesh test, tests/test_mpmd_mesh.py:71).
Routing here is capacity based so that every shape in the captured step is static:

    probs   = softmax(x W_r^T)                       [T, E]
    top-k   → expert ids, weights renormalised over the k picks; aux = E * Σ_e f_e · P_e (load balancing)
    dispatch: token t's copy for expert e goes to slot (number of earlier tokens routed to e); copies beyond
              the capacity C are dropped                → buffer [E, C, d]
    all-to-all over the expert axis: rank r keeps experts [r·E_l, (r+1)·E_l)           → [E_l, ep·C, d]
    expert FFN (SwiGLU) per local expert — equal-sized groups, one tcgen05 GEMM per expert and projection
    all-to-all back, combine: y_t = Σ_k w_{t,k} · out[e_{t,k}, slot_{t,k}]

``b200tp::all_to_all`` is the collective (its transpose is itself); the permutations are index ops whose
autograd gives the matching scatter/gather in backward.  On GPUs with fused collectives enabled, dispatch and
combine run as peer-memory kernels (``jaxpp_b200.parallel.fused_moe``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ..ops import core as ops
from . import tp as tpmod

_lib = torch.library.Library("b200moe", "DEF")


def _all_to_all_impl(x: Tensor, axis: str) -> Tensor:
    """x: [n, ...] — block q goes to rank q of the axis; returns [n, ...] with block q received from rank q."""
    n = tpmod.axis_size(axis)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=tpmod._group(axis))
    return out


_lib.define("all_to_all(Tensor x, str axis) -> Tensor")
_lib.impl("all_to_all", _all_to_all_impl, "CompositeExplicitAutograd")
torch.library.register_fake("b200moe::all_to_all", lambda x, axis: torch.empty_like(x))
torch.library.register_autograd(
    "b200moe::all_to_all",
    lambda ctx, g: (torch.ops.b200moe.all_to_all(g.contiguous(), ctx.axis), None),
    setup_context=lambda ctx, inputs, output: setattr(ctx, "axis", inputs[1]),
)


def route(x: Tensor, w_router: Tensor, top_k: int):
    """Returns (expert ids [T,k] int64, weights [T,k] fp32, aux loss scalar fp32)."""
    logits = ops.linear(x, w_router, None).float()
    probs = torch.softmax(logits, dim=-1)
    top_v, top_i = probs.topk(top_k, dim=-1)
    weights = top_v / top_v.sum(-1, keepdim=True)
    E = w_router.shape[0]
    hits = torch.nn.functional.one_hot(top_i, E).sum(1).to(torch.float32)  # [T, E]
    frac = hits.mean(0) / top_k
    aux = E * (frac.detach() * probs.mean(0)).sum()
    return top_i, weights, aux


def slots_for(top_i: Tensor, n_experts: int, capacity: int):
    """Flat destination index (expert * C + position) of every (token, pick); dropped picks map to the dump
    row ``E * C``.  Position = how many earlier (token-major) picks chose the same expert."""
    T, k = top_i.shape
    flat = top_i.reshape(-1)
    onehot = torch.nn.functional.one_hot(flat, n_experts)
    pos = (onehot.cumsum(0) - 1).gather(1, flat[:, None]).squeeze(1)
    keep = pos < capacity
    dest = torch.where(keep, flat * capacity + pos, torch.full_like(flat, n_experts * capacity))
    return dest, keep


def dispatch(x: Tensor, dest: Tensor, n_experts: int, capacity: int, top_k: int) -> Tensor:
    """[T, d] → [E, C, d]; every kept (token, pick) copies the token's row into its slot."""
    d = x.shape[-1]
    src = x.repeat_interleave(top_k, dim=0)
    buf = torch.zeros(n_experts * capacity + 1, d, dtype=x.dtype, device=x.device)
    buf = buf.index_add(0, dest, src)
    return buf[:-1].view(n_experts, capacity, d)


def combine(y_buf: Tensor, dest: Tensor, weights: Tensor, top_k: int) -> Tensor:
    """[E, C, d] → [T, d]: weighted sum of each token's picks (dropped picks contribute zero)."""
    E, C, d = y_buf.shape
    flat = torch.cat([y_buf.reshape(E * C, d), torch.zeros(1, d, dtype=y_buf.dtype, device=y_buf.device)], 0)
    picked = flat.index_select(0, dest).view(-1, top_k, d)
    return (picked.float() * weights.unsqueeze(-1)).sum(1).to(y_buf.dtype)


def expert_ffn(x: Tensor, w_up: Tensor, w_down: Tensor) -> Tensor:
    """x: [E_l, M, d]; w_up: [E_l, 2F, d] ([gate | up]); w_down: [E_l, d, F]"""
    outs = []
    for e in range(x.shape[0]):
        h = ops.swiglu(ops.linear(x[e], w_up[e], None))
        outs.append(ops.linear(h, w_down[e], None))
    return torch.stack(outs, 0)


def moe_ffn(x: Tensor, p: dict, n_experts: int, top_k: int, capacity_factor: float, ep: int, ep_axis: str):
    """Full MoE feed-forward on this device's tokens ``x`` [T, d].  Returns (y [T, d], aux loss)."""
    T, d = x.shape
    capacity = int(-(-T * top_k * capacity_factor // n_experts))
    capacity = (capacity + 7) // 8 * 8
    top_i, weights, aux = route(x, p["router"], top_k)
    dest, _ = slots_for(top_i, n_experts, capacity)
    buf = dispatch(x, dest, n_experts, capacity, top_k)                        # [E, C, d]
    e_local = n_experts // ep
    if ep > 1:
        buf = torch.ops.b200moe.all_to_all(buf.view(ep, e_local * capacity, d), ep_axis)   # block q from rank q
        buf = buf.view(ep, e_local, capacity, d).transpose(0, 1).reshape(e_local, ep * capacity, d)
    y = expert_ffn(buf, p["w_up"], p["w_down"])                                # [E_l, ep*C, d]
    if ep > 1:
        y = y.view(e_local, ep, capacity, d).transpose(0, 1).reshape(ep, e_local * capacity, d)
        y = torch.ops.b200moe.all_to_all(y.contiguous(), ep_axis)
    y = y.reshape(n_experts, capacity, d)
    return combine(y, dest, weights, top_k), aux
