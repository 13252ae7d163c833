"""Context parallelism: attention over a sequence that is split across the ranks of a mesh axis (ring attention).

Rank ``r`` of ``n`` holds the ``r``-th contiguous chunk of every sequence: ``q, k, v`` are ``[batch, s_local, heads,
head_dim]``.  The key / value chunks travel once around the ring; every rank runs the flash-attention kernel of
``ops.attention`` on its queries against the chunk it currently holds and merges the partial results through their
log-sum-exp, so no rank ever materialises more than two chunks of keys and values.  With ``causal`` a chunk from a
later rank is skipped (fully masked), the own chunk is causal, earlier chunks are full.  The backward pass repeats the
ring: the chunk's ``dk, dv`` accumulators travel with it and arrive home after ``n`` hops, ``dq`` stays.

    o = context.ring_attention(q, k, v, causal, scale, axis)          # differentiable

Transfers are point-to-point operations on the axis' own process group (NCCL on GPUs, gloo on CPU), posted before the
block's attention kernel so that they overlap it.  The reference has no context parallelism (its long-context advice
is rematerialisation and offloading, PERF_GUIDE.md:51-54); everything else in a transformer block is token-local, so a
model shards its sequence over the axis, uses this op for attention and sums parameter gradients over the axis as it
does for data parallelism.

Layouts.  ``contiguous``: rank ``r`` holds chunk ``r``; under ``causal`` rank ``r`` computes ``r + 1`` of the ``n``
blocks, so the last rank paces the ring.  ``zigzag``: the sequence is cut into ``2n`` pieces and rank ``r`` holds pieces
``r`` and ``2n-1-r`` (concatenated); then every rank computes the causal block on its own chunk plus, per other rank,
exactly half a block (all its queries against the earlier rank's first piece, or its second piece's queries against
the later rank's whole chunk), which balances the causal work.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ..ops import core as ops
from . import tp as tpmod

_lib = torch.library.Library("b200cp", "DEF")


def _ring(axis: str):
    """(n, r, global rank of the next / previous rank on the ring, process group)"""
    from ..mesh import MpmdMesh

    mesh = MpmdMesh.current()
    n = mesh.shape[axis]
    if n == 1:
        return 1, 0, None, None, None
    peers = [d.process_index for d in mesh.peers_along(axis)]
    r = mesh.axis_index(axis)
    return n, r, peers[(r + 1) % n], peers[(r - 1) % n], mesh.axis_group(axis)


def _rotate(tensors: list, nxt: int, prv: int, group) -> tuple[list, list]:
    """Post the sends of ``tensors`` to the next rank and the receives from the previous one; returns the receive
    buffers and the requests to wait for."""
    bufs = [torch.empty_like(t) for t in tensors]
    p2p = [dist.P2POp(dist.isend, t.contiguous(), nxt, group) for t in tensors]
    p2p += [dist.P2POp(dist.irecv, b, prv, group) for b in bufs]
    return bufs, dist.batch_isend_irecv(p2p)


def _wait(reqs: list) -> None:
    for q in reqs:
        q.wait()


def _merge(out: Tensor, lse: Tensor, o_i: Tensor, lse_i: Tensor, rows: slice) -> None:
    """Fold a block's (o_i, lse_i) for query rows ``rows`` into the running fp32 output / log-sum-exp, in place."""
    old = lse[:, :, rows]
    new = torch.logaddexp(old, lse_i)
    w_old = torch.exp(old - new).transpose(1, 2).unsqueeze(-1)                             # [B, S, H, 1]
    w_new = torch.exp(lse_i - new).transpose(1, 2).unsqueeze(-1)
    out[:, rows] = out[:, rows] * w_old + o_i.float() * w_new
    lse[:, :, rows] = new


def _fwd_impl(q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float, axis: str, layout: str = "contiguous"):
    n, r, nxt, prv, group = _ring(axis)
    if n == 1:
        return ops.attention(q, k, v, causal, scale)
    if layout not in ("contiguous", "zigzag"):
        raise ValueError(f"unknown sequence layout {layout!r}")
    zigzag = causal and layout == "zigzag"
    half = q.shape[1] // 2
    everything, back = slice(None), slice(half, None)
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)                       # [B, S, H, D]
    lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("-inf"), dtype=torch.float32, device=q.device)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    for step in range(n):
        src = (r - step) % n                      # owner of the chunk held now
        reqs = None
        if step < n - 1:
            (k_nxt, v_nxt), reqs = _rotate([k_cur, v_cur], nxt, prv, group)
        if zigzag and src < r:      # an earlier rank: only its first piece precedes my queries, and all of them
            o_i, lse_i = ops.attention(q, k_cur[:, :half].contiguous(), v_cur[:, :half].contiguous(), False, scale)
            _merge(out, lse, o_i, lse_i, everything)
        elif zigzag and src > r:    # a later rank: both its pieces precede my second piece and follow my first
            o_i, lse_i = ops.attention(q[:, half:].contiguous(), k_cur, v_cur, False, scale)
            _merge(out, lse, o_i, lse_i, back)
        elif not (causal and src > r):
            o_i, lse_i = ops.attention(q, k_cur, v_cur, causal and src == r, scale)
            _merge(out, lse, o_i, lse_i, everything)
        if reqs is not None:
            _wait(reqs)
            k_cur, v_cur = k_nxt, v_nxt
    return out.to(q.dtype), lse


def _bwd_impl(do: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, causal: bool, scale: float, axis: str,
              layout: str = "contiguous"):
    n, r, nxt, prv, group = _ring(axis)
    if n == 1:
        return ops.attention_bwd(do, q, k, v, o, lse, causal, scale)
    zigzag = causal and layout == "zigzag"
    half = q.shape[1] // 2
    do = do.contiguous()
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    dk_cur = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
    dv_cur = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
    for step in range(n):
        src = (r - step) % n
        kv_reqs = None
        if step < n - 1:                          # the chunk itself is needed by n - 1 more ranks
            (k_nxt, v_nxt), kv_reqs = _rotate([k_cur, v_cur], nxt, prv, group)
        if zigzag and src < r:
            dq_i, dk_i, dv_i = ops.attention_bwd(do, q, k_cur[:, :half].contiguous(), v_cur[:, :half].contiguous(), o, lse,
                                                 False, scale)
            dq += dq_i.float()
            dk_cur[:, :half] += dk_i.float()
            dv_cur[:, :half] += dv_i.float()
        elif zigzag and src > r:
            dq_i, dk_i, dv_i = ops.attention_bwd(do[:, half:].contiguous(), q[:, half:].contiguous(), k_cur, v_cur,
                                                 o[:, half:].contiguous(), lse[:, :, half:].contiguous(), False, scale)
            dq[:, half:] += dq_i.float()
            dk_cur += dk_i.float()
            dv_cur += dv_i.float()
        elif not (causal and src > r):
            # the global o and lse make every block's probabilities and row sums those of the whole sequence
            dq_i, dk_i, dv_i = ops.attention_bwd(do, q, k_cur, v_cur, o, lse, causal and src == r, scale)
            dq += dq_i.float()
            dk_cur += dk_i.float()
            dv_cur += dv_i.float()
        # the accumulators follow the chunk; after n hops they are back at its owner
        (dk_nxt, dv_nxt), g_reqs = _rotate([dk_cur, dv_cur], nxt, prv, group)
        if kv_reqs is not None:
            _wait(kv_reqs)
            k_cur, v_cur = k_nxt, v_nxt
        _wait(g_reqs)
        dk_cur, dv_cur = dk_nxt, dv_nxt
    return dq.to(q.dtype), dk_cur.to(k.dtype), dv_cur.to(v.dtype)


_lib.define("ring_attention(Tensor q, Tensor k, Tensor v, bool causal, float scale, str axis, str layout=\"contiguous\")"
            " -> (Tensor, Tensor)")
_lib.impl("ring_attention", _fwd_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200cp::ring_attention",
    lambda q, k, v, causal, scale, axis, layout="contiguous": (torch.empty_like(q),
                                          q.new_empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32)))

_lib.define("ring_attention_bwd(Tensor do, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, bool causal, float scale,"
            " str axis, str layout=\"contiguous\") -> (Tensor, Tensor, Tensor)")
_lib.impl("ring_attention_bwd", _bwd_impl, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200cp::ring_attention_bwd",
    lambda do, q, k, v, o, lse, causal, scale, axis, layout="contiguous": (torch.empty_like(q), torch.empty_like(k),
                                                                           torch.empty_like(v)))


def _setup(ctx, inputs, output):
    q, k, v, causal, scale, axis, layout = inputs
    ctx.save_for_backward(q, k, v, output[0], output[1])
    ctx.causal, ctx.scale, ctx.axis, ctx.layout = causal, scale, axis, layout


def _backward(ctx, do, dlse):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = torch.ops.b200cp.ring_attention_bwd(do.contiguous(), q, k, v, o, lse, ctx.causal, ctx.scale, ctx.axis,
                                                     ctx.layout)
    return dq, dk, dv, None, None, None, None


torch.library.register_autograd("b200cp::ring_attention", _backward, setup_context=_setup)


def ring_attention(q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float, axis: str,
                   layout: str = "contiguous") -> Tensor:
    """Attention of this rank's queries over the whole sequence held by the ranks of ``axis``; ``q, k, v`` are this
    rank's ``[batch, s_local, heads, head_dim]`` chunk in the given ``layout`` (grouped-query heads as in
    ``ops.attention``)."""
    return torch.ops.b200cp.ring_attention(q, k, v, causal, float(scale), axis, layout)[0]


def local_sequence_slice(x: Tensor, axis: str, dim: int = 1, layout: str = "contiguous") -> Tensor:
    """This rank's chunk of ``x`` along the sequence dimension ``dim``: chunk ``r`` of ``n``, or for ``zigzag`` pieces
    ``r`` and ``2n-1-r`` of ``2n`` concatenated."""
    n = tpmod.axis_size(axis)
    if n == 1:
        return x
    r = tpmod.axis_rank(axis)
    if layout == "zigzag":
        s = x.shape[dim] // (2 * n)
        return torch.cat([x.narrow(dim, r * s, s), x.narrow(dim, (2 * n - 1 - r) * s, s)], dim=dim)
    s = x.shape[dim] // n
    return x.narrow(dim, r * s, s)

def _register_direct_calls():
    """Generated task code calls these implementations without the dispatcher (see ops.core.DIRECT)."""
    from ..ops import core as _core

    _core.DIRECT[torch.ops.b200cp.ring_attention.default] = _fwd_impl
    _core.DIRECT[torch.ops.b200cp.ring_attention_bwd.default] = _bwd_impl


_register_direct_calls()
