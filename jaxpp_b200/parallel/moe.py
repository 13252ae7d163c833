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

With expert parallelism the two exchanges are the ops ``b200moe::dispatch_a2a`` (permutation into slots +
all-to-all) and ``b200moe::combine_a2a`` (all-to-all back + weighted gather-sum); each is the other's
transpose, which is how their backward is written.  On GPUs with fused collectives enabled they run as one
peer-memory kernel each (``jaxpp_b200.parallel.fused_moe``), otherwise as index ops around
``b200moe::all_to_all`` (NCCL / gloo).
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


# ---- dispatch / combine fused with the expert-parallel exchange ------------------------------------------------------
def _use_fused(x: Tensor) -> bool:
    from ..utils import config

    if not (x.is_cuda and config.use_fused_collectives.value and config.use_native_kernels.value):
        return False
    from . import fused_moe

    return fused_moe.supported(x)


def _dispatch_a2a_impl(x, dest, scale, n_experts: int, capacity: int, top_k: int, axis: str):
    """x [T, d]; dest [T*k] slot (expert * C + position, E*C = dropped); scale [T*k] or None.
    Returns [E_l, ep*C, d]: for every local expert, the slots of rank 0's tokens, then rank 1's, ..."""
    ep = tpmod.axis_size(axis)
    d = x.shape[-1]
    e_local = n_experts // ep
    if ep > 1 and _use_fused(x):
        from . import fused_moe

        n_slots = n_experts * capacity
        picks = torch.arange(dest.numel(), device=x.device, dtype=torch.int32)
        inv = torch.full((n_slots + 1,), -1, dtype=torch.int32, device=x.device)
        inv[dest] = picks // top_k
        slot_scale = None
        if scale is not None:
            slot_scale = torch.zeros(n_slots + 1, dtype=torch.float32, device=x.device)
            slot_scale[dest] = scale.float()
        return fused_moe.dispatch(x, inv, slot_scale, n_experts, capacity, axis)
    src = x.repeat_interleave(top_k, dim=0)
    if scale is not None:
        src = (src.float() * scale.float().unsqueeze(-1)).to(x.dtype)
    buf = torch.zeros(n_experts * capacity + 1, d, dtype=x.dtype, device=x.device)
    buf = buf.index_add(0, dest, src)[:-1]
    if ep == 1:
        return buf.view(n_experts, capacity, d)
    buf = _all_to_all_impl(buf.view(ep, e_local * capacity, d), axis)   # block q from rank q
    return buf.view(ep, e_local, capacity, d).transpose(0, 1).reshape(e_local, ep * capacity, d)


def _combine_a2a_impl(y, dest, weights, n_experts: int, capacity: int, top_k: int, axis: str, want_picked: bool):
    """y [E_l, ep*C, d] -> (out [T, d], picked [T*k, d] or an empty tensor)."""
    ep = tpmod.axis_size(axis)
    d = y.shape[-1]
    e_local = n_experts // ep
    T = dest.numel() // top_k
    if ep > 1 and _use_fused(y):
        from . import fused_moe

        out, picked = fused_moe.combine(y, dest.to(torch.int32), None if weights is None else weights.float().contiguous(),
                                        n_experts, capacity, top_k, axis, want_picked)
        return out, picked if picked is not None else y.new_empty(0)
    if ep > 1:
        y = y.view(e_local, ep, capacity, d).transpose(0, 1).reshape(ep, e_local * capacity, d)
        y = _all_to_all_impl(y.contiguous(), axis)
    flat = torch.cat([y.reshape(n_experts * capacity, d), torch.zeros(1, d, dtype=y.dtype, device=y.device)], 0)
    picked = flat.index_select(0, dest)
    w = weights.float() if weights is not None else torch.ones(dest.numel(), dtype=torch.float32, device=y.device)
    out = (picked.view(T, top_k, d).float() * w.view(T, top_k, 1)).sum(1).to(y.dtype)
    return out, picked if want_picked else y.new_empty(0)


_lib.define("dispatch_a2a(Tensor x, Tensor dest, Tensor? scale, int n_experts, int capacity, int top_k, str axis) -> Tensor")
_lib.impl("dispatch_a2a", _dispatch_a2a_impl, "CompositeExplicitAutograd")
_lib.define("combine_a2a(Tensor y, Tensor dest, Tensor? weights, int n_experts, int capacity, int top_k, str axis, "
            "bool want_picked) -> (Tensor, Tensor)")
_lib.impl("combine_a2a", _combine_a2a_impl, "CompositeExplicitAutograd")


def _dispatch_fake(x, dest, scale, n_experts, capacity, top_k, axis):
    ep = tpmod.axis_size(axis)
    return x.new_empty(n_experts // ep, ep * capacity, x.shape[-1])


def _combine_fake(y, dest, weights, n_experts, capacity, top_k, axis, want_picked):
    T = dest.numel() // top_k
    return y.new_empty(T, y.shape[-1]), y.new_empty((dest.numel(), y.shape[-1]) if want_picked else (0,))


torch.library.register_fake("b200moe::dispatch_a2a", _dispatch_fake)
torch.library.register_fake("b200moe::combine_a2a", _combine_fake)


def _dispatch_setup(ctx, inputs, output):
    _, dest, scale, ctx.n_experts, ctx.capacity, ctx.top_k, ctx.axis = inputs
    ctx.save_for_backward(dest, scale)


def _dispatch_bwd(ctx, g):
    # the transpose of "scatter rows into slots, scaled" is "gather-sum the slots of each token, scaled";
    # no gradient flows to the scale (it is only used inside the backward of combine)
    dest, scale = ctx.saved_tensors
    dx, _ = torch.ops.b200moe.combine_a2a(g.contiguous(), dest, scale, ctx.n_experts, ctx.capacity, ctx.top_k, ctx.axis, False)
    return dx, None, None, None, None, None, None


def _combine_setup(ctx, inputs, output):
    _, dest, weights, ctx.n_experts, ctx.capacity, ctx.top_k, ctx.axis, ctx.want_picked = inputs
    ctx.has_weights = weights is not None
    ctx.save_for_backward(dest, weights, output[1])


def _combine_bwd(ctx, g_out, g_picked):
    dest, weights, picked = ctx.saved_tensors
    g_out = g_out.contiguous()
    dy = torch.ops.b200moe.dispatch_a2a(g_out, dest, weights, ctx.n_experts, ctx.capacity, ctx.top_k, ctx.axis)
    dw = None
    if ctx.has_weights and ctx.needs_input_grad[2]:
        if not ctx.want_picked:
            raise RuntimeError("combine_a2a needs want_picked=True to differentiate with respect to the weights")
        T = g_out.shape[0]
        dw = (picked.view(T, ctx.top_k, -1).float() * g_out.float().unsqueeze(1)).sum(-1).reshape(-1).to(weights.dtype)
    return dy, None, dw, None, None, None, None, None


torch.library.register_autograd("b200moe::dispatch_a2a", _dispatch_bwd, setup_context=_dispatch_setup)
torch.library.register_autograd("b200moe::combine_a2a", _combine_bwd, setup_context=_combine_setup)


def _route_ref(logits: Tensor, top_k: int):
    """(expert ids [T,k] int64, weights [T,k] fp32, probabilities [T,E] fp32, picks per expert [E] fp32)"""
    probs = torch.softmax(logits.float(), dim=-1)
    top_v, top_i = probs.topk(top_k, dim=-1)
    weights = top_v / top_v.sum(-1, keepdim=True)
    hits = torch.nn.functional.one_hot(top_i, logits.shape[-1]).sum((0, 1)).to(torch.float32)
    return top_i, weights, probs, hits


def _router_impl(logits: Tensor, top_k: int):
    from ..ops import core as _core

    if _core._use_native(logits) and logits.dtype in (torch.float32, torch.bfloat16) and logits.shape[-1] <= 64 and top_k <= 8:
        import ctypes

        from ..ops import native

        lib = native.load()
        p, i = ctypes.c_void_p, ctypes.c_int
        lib.jpb_router.argtypes = [i, p, p, p, p, p, p, i, i, i, p]
        lg = logits.contiguous()
        T, E = lg.shape
        dev = lg.device
        probs = torch.empty(T, E, dtype=torch.float32, device=dev)
        top_i = torch.empty(T, top_k, dtype=torch.int64, device=dev)
        weights = torch.empty(T, top_k, dtype=torch.float32, device=dev)
        stats = torch.empty(2, E, dtype=torch.float32, device=dev)
        native._check(lib.jpb_router(0 if lg.dtype == torch.float32 else 1, lg.data_ptr(), probs.data_ptr(), top_i.data_ptr(),
                                     weights.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(), T, E, top_k,
                                     native._stream()), "jpb_router")
        return top_i, weights, probs, stats[1]
    return _route_ref(logits, top_k)


_lib.define("router(Tensor logits, int top_k) -> (Tensor, Tensor, Tensor, Tensor)")
_lib.impl("router", _router_impl, "CompositeExplicitAutograd")


def _router_fake(logits, top_k):
    T, E = logits.shape
    f32 = dict(dtype=torch.float32, device=logits.device)
    return (torch.empty(T, top_k, dtype=torch.int64, device=logits.device), torch.empty(T, top_k, **f32),
            torch.empty(T, E, **f32), torch.empty(E, **f32))


torch.library.register_fake("b200moe::router", _router_fake)


def _router_setup(ctx, inputs, output):
    ctx.save_for_backward(output[0], output[2])
    ctx.in_dtype = inputs[0].dtype


def _router_bwd(ctx, g_idx, g_w, g_probs, g_hits):
    """weights_j = p_{i_j} / S with S the sum of the picked probabilities; probs = softmax(logits)."""
    top_i, probs = ctx.saved_tensors
    dp = g_probs.float() if g_probs is not None else torch.zeros_like(probs)
    if g_w is not None:
        pv = probs.gather(1, top_i)
        s = pv.sum(-1, keepdim=True)
        gw = g_w.float()
        d_pv = gw / s - (gw * pv).sum(-1, keepdim=True) / (s * s)
        dp = dp.scatter_add(1, top_i, d_pv)
    dlogits = probs * (dp - (dp * probs).sum(-1, keepdim=True))
    return dlogits.to(ctx.in_dtype), None


torch.library.register_autograd("b200moe::router", _router_bwd, setup_context=_router_setup)


def route(x: Tensor, w_router: Tensor, top_k: int):
    """Returns (expert ids [T,k] int64, weights [T,k] fp32, aux loss scalar fp32).  Softmax, top-k, renormalised
    weights and the load-balancing statistics come from one kernel on the GPU (``b200moe::router``)."""
    logits = ops.linear(x, w_router, None)
    top_i, weights, probs, hits = torch.ops.b200moe.router(logits, top_k)
    E = w_router.shape[0]
    frac = hits / (top_i.shape[0] * top_k)
    aux = E * (frac.detach() * probs.mean(0)).sum()
    return top_i, weights, aux


def slots_for(top_i: Tensor, n_experts: int, capacity: int):
    """Flat destination index (expert * C + position) of every (token, pick); dropped picks map to the dump
    row ``E * C``.  Position = how many earlier (token-major) picks chose the same expert."""
    dest, keep, _ = slots_and_counts(top_i, n_experts, capacity)
    return dest, keep


def slots_and_counts(top_i: Tensor, n_experts: int, capacity: int):
    """:func:`slots_for` plus ``counts`` [E] int32: how many slots of each expert this device's tokens fill."""
    flat = top_i.reshape(-1)
    # running count of picks per expert, scanned along the CONTIGUOUS dimension of an [E, picks] int32 matrix: the same
    # scan down the rows of a [picks, E] int64 one-hot matrix took 3.2 ms per call on the GPU (15 % of a Mixtral step)
    onehot_t = (flat[None, :] == torch.arange(n_experts, device=flat.device, dtype=flat.dtype)[:, None]).to(torch.int32)
    running = onehot_t.cumsum(1, dtype=torch.int32)                   # [E, picks]
    pos = (running.gather(0, flat[None, :]).squeeze(0) - 1).to(flat.dtype)
    keep = pos < capacity
    dest = torch.where(keep, flat * capacity + pos, torch.full_like(flat, n_experts * capacity))
    counts = running[:, -1].clamp(max=capacity).to(torch.int32)
    return dest, keep, counts


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


def expert_ffn(x: Tensor, w_up: Tensor, w_down: Tensor, counts: Tensor | None = None, seg_rows: int = 0) -> Tensor:
    """x: [E_l, M, d]; w_up: [E_l, 2F, d] ([gate | up]); w_down: [E_l, d, F].  Every local expert has room for the
    same number of slots, so each projection is one grouped tcgen05 GEMM over all local experts.  ``counts``
    [E_l, M / seg_rows] says how many slots at the start of each ``seg_rows``-slot segment are filled (the others hold
    zeros): the GEMMs of the forward and of both gradients skip the tiles made of empty slots."""
    E_l, M, d = x.shape
    h = ops.swiglu(ops.linear_batched(x, w_up, counts, seg_rows).view(E_l * M, -1))
    return ops.linear_batched(h.view(E_l, M, -1), w_down, counts, seg_rows)


def moe_ffn(x: Tensor, p: dict, n_experts: int, top_k: int, capacity_factor: float, ep: int, ep_axis: str):
    """Full MoE feed-forward on this device's tokens ``x`` [T, d].  Returns (y [T, d], aux loss)."""
    T, d = x.shape
    capacity = int(-(-T * top_k * capacity_factor // n_experts))
    capacity = (capacity + 7) // 8 * 8
    from ..utils import config

    top_i, weights, aux = route(x, p["router"], top_k)
    dest, _, counts = slots_and_counts(top_i, n_experts, capacity)
    if config.moe_skip_empty_slots.value <= 0:
        counts = None
    if ep > 1:
        buf = torch.ops.b200moe.dispatch_a2a(x, dest, None, n_experts, capacity, top_k, ep_axis)   # [E_l, ep*C, d]
        if counts is not None:
            # every rank tells the owner of each expert how many of its C slots it filled: [ep (source), E_l] -> [E_l, ep]
            counts = torch.ops.b200moe.all_to_all(counts.view(ep, n_experts // ep), ep_axis).t().contiguous()
        y = expert_ffn(buf, p["w_up"], p["w_down"], counts, capacity)
        out, _ = torch.ops.b200moe.combine_a2a(y, dest, weights.reshape(-1), n_experts, capacity, top_k, ep_axis, True)
        return out, aux
    buf = dispatch(x, dest, n_experts, capacity, top_k)                        # [E, C, d]
    y = expert_ffn(buf, p["w_up"], p["w_down"], None if counts is None else counts.view(n_experts, 1), capacity)
    return combine(y.reshape(n_experts, capacity, d), dest, weights, top_k), aux

def _register_direct_calls():
    """Generated task code calls these implementations without the dispatcher (see ops.core.DIRECT)."""
    from ..ops import core as _core

    _core.DIRECT[torch.ops.b200moe.all_to_all.default] = _all_to_all_impl
    _core.DIRECT[torch.ops.b200moe.dispatch_a2a.default] = _dispatch_a2a_impl
    _core.DIRECT[torch.ops.b200moe.combine_a2a.default] = _combine_a2a_impl
    _core.DIRECT[torch.ops.b200moe.router.default] = _router_impl


_register_direct_calls()
