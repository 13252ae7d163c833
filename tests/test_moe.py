"""Mixture-of-experts building blocks on CPU: routing, capacity slots, dispatch / combine and their transposes."""
import torch

import jaxpp_b200 as jp
from jaxpp_b200.parallel import moe


def _mesh():
    return jp.MpmdMesh.create({"mpmd": 1, "data": 1, "model": 1}, kind="cpu", multi_process=False)


def _routing(T=24, E=4, k=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    top_i = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    return top_i


def test_slots_are_unique_and_capacity_bounded():
    top_i = _routing(T=40, E=4, k=2)
    C = 8
    dest, keep = moe.slots_for(top_i, 4, C)
    kept = dest[keep]
    assert kept.unique().numel() == kept.numel()          # no two picks share a slot
    assert (kept // C == top_i.reshape(-1)[keep]).all()   # a slot belongs to the expert that was picked
    assert (dest[~keep] == 4 * C).all() and (~keep).any()  # picks beyond the capacity go to the dump row
    # positions are assigned in token order
    e0 = (top_i.reshape(-1) == 0).nonzero().squeeze(1)
    assert (dest[e0[:C]] == torch.arange(C)).all()


def test_slot_counts_and_grouped_linear_with_counts():
    """The per-expert counts of filled slots (what lets the grouped GEMMs skip unused capacity) against a direct count,
    and the grouped linear op with counts against the one without: zero rows give zero products, so results and
    gradients must be identical (on CPU the counts are ignored; on the GPU they select the skipping kernels)."""
    from jaxpp_b200.ops import core as ops

    top_i = _routing(T=40, E=4, k=2, seed=3)
    C = 16
    dest, keep, counts = moe.slots_and_counts(top_i, 4, C)
    flat = top_i.reshape(-1)
    assert counts.dtype == torch.int32
    assert counts.tolist() == [min(C, int((flat == e).sum())) for e in range(4)]
    assert int(keep.sum()) == int(counts.sum())
    d2, k2 = moe.slots_for(top_i, 4, C)
    assert torch.equal(d2, dest) and torch.equal(k2, keep)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(40, 8, generator=g)
    buf = moe.dispatch(x, dest, 4, C, 2)                                  # [E, C, d], unused slots are zero
    live = torch.arange(C)[None, :] < counts[:, None]
    assert (buf[~live] == 0).all()
    w = torch.randn(4, 6, 8, generator=g, requires_grad=True)
    bx = buf.clone().requires_grad_(True)
    y0 = ops.linear_batched(bx, w)
    g0 = torch.autograd.grad(y0.square().sum(), [bx, w])
    y1 = ops.linear_batched(bx, w, counts.view(4, 1), C)
    g1 = torch.autograd.grad(y1.square().sum(), [bx, w])
    assert torch.equal(y0, y1) and all(torch.equal(a, b) for a, b in zip(g0, g1))


def test_fused_ops_match_index_ops_and_are_transposes():
    T, E, k, d, C = 24, 4, 2, 16, 8
    top_i = _routing(T, E, k, seed=1)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, d, generator=g, dtype=torch.float64)
    w = torch.rand(T, k, generator=g, dtype=torch.float64)
    with _mesh():
        dest, _ = moe.slots_for(top_i, E, C)
        buf_ref = moe.dispatch(x, dest, E, C, k)
        buf = torch.ops.b200moe.dispatch_a2a(x, dest, None, E, C, k, "data")
        torch.testing.assert_close(buf, buf_ref)
        y = torch.randn(E, C, d, generator=g, dtype=torch.float64)
        out_ref = moe.combine(y, dest, w, k)
        out, picked = torch.ops.b200moe.combine_a2a(y, dest, w.reshape(-1), E, C, k, "data", True)
        torch.testing.assert_close(out, out_ref, rtol=1e-5, atol=1e-5)
        assert picked.shape == (T * k, d)

        # <dispatch(x), y> == <x, combine(y)> with unit weights: the two ops are transposes of each other
        ones = torch.ones(T * k, dtype=torch.float64)
        lhs = (buf * y).sum()
        rhs = (x * torch.ops.b200moe.combine_a2a(y, dest, ones, E, C, k, "data", False)[0]).sum()
        torch.testing.assert_close(lhs, rhs, rtol=1e-5, atol=1e-5)  # combine accumulates in fp32

        # autograd of the ops against autograd of the index ops
        xr, yr, wr = x.clone().requires_grad_(True), y.clone().requires_grad_(True), w.clone().requires_grad_(True)
        loss_ref = (moe.combine(moe.dispatch(xr, dest, E, C, k) * 2 + yr, dest, wr, k) ** 2).sum()
        g_ref = torch.autograd.grad(loss_ref, [xr, yr, wr])
        xo, yo, wo = x.clone().requires_grad_(True), y.clone().requires_grad_(True), w.clone().requires_grad_(True)
        b = torch.ops.b200moe.dispatch_a2a(xo, dest, None, E, C, k, "data")
        o, _ = torch.ops.b200moe.combine_a2a(b * 2 + yo, dest, wo.reshape(-1), E, C, k, "data", True)
        g_new = torch.autograd.grad((o ** 2).sum(), [xo, yo, wo])
        for a, b_ in zip(g_ref, g_new):
            torch.testing.assert_close(b_, a, rtol=1e-4, atol=1e-5)


def test_moe_ffn_drops_and_aux_loss():
    torch.manual_seed(0)
    T, d, F, E, k = 32, 16, 24, 4, 2
    p = {"router": torch.randn(E, d) * 0.1, "w_up": torch.randn(E, 2 * F, d) * 0.1, "w_down": torch.randn(E, d, F) * 0.1}
    x = torch.randn(T, d)
    with _mesh():
        y, aux = moe.moe_ffn(x, p, E, k, 4.0, 1, "data")       # capacity large enough: nothing is dropped
        # dense oracle: every token through its k experts
        probs = torch.softmax(x @ p["router"].t(), -1)
        tv, ti = probs.topk(k, -1)
        tw = tv / tv.sum(-1, keepdim=True)
        ref = torch.zeros_like(x)
        for t in range(T):
            for j in range(k):
                e = int(ti[t, j])
                h = x[t] @ p["w_up"][e].t()
                h = torch.nn.functional.silu(h[:F]) * h[F:]
                ref[t] += tw[t, j] * (h @ p["w_down"][e].t())
        torch.testing.assert_close(y, ref, rtol=1e-4, atol=1e-5)
        assert aux.item() > 0
        y_small, _ = moe.moe_ffn(x, p, E, k, 0.25, 1, "data")  # tight capacity: some picks are dropped
        assert not torch.allclose(y_small, ref)


def test_router_op_backward_matches_autograd_of_the_composition():
    torch.manual_seed(3)
    T, E, k = 50, 8, 2
    logits = torch.randn(T, E, dtype=torch.float64)
    gw, gp = torch.randn(T, k, dtype=torch.float64), torch.randn(T, E, dtype=torch.float64)

    def loss(fn, lg):
        top_i, w, probs, hits = fn(lg, k)
        return (w.double() * gw).sum() + (probs.double() * gp).sum(), top_i, hits

    a = logits.clone().requires_grad_(True)
    la, ia, ha = loss(moe._route_ref, a)
    (ga,) = torch.autograd.grad(la, [a])
    b = logits.clone().requires_grad_(True)
    lb, ib, hb = loss(torch.ops.b200moe.router, b)
    (gb,) = torch.autograd.grad(lb, [b])
    assert torch.equal(ia, ib) and torch.equal(ha, hb) and hb.sum().item() == T * k
    torch.testing.assert_close(gb, ga, rtol=1e-5, atol=1e-6)
