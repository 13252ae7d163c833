"""Numerics of every native sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from jaxpp_b200.ops import native as n

    n.load()  # fails loudly if the library was not built
    yield n
    torch.cuda.synchronize()
    assert n.read_status() == 0, "a kernel reported a bounded-wait time-out or a bad argument"


def rnd(*shape, dtype=torch.bfloat16, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dtype)


def close(got, ref, rtol, atol):
    torch.testing.assert_close(got.float(), ref.float(), rtol=rtol, atol=atol)


GEMM_SHAPES = [
    (128, 256, 64), (256, 512, 128), (384, 768, 192), (130, 264, 72),  # ragged M/N/K tails
    (1024, 1600, 6400), (512, 11008, 4096), (2048, 4096, 5504), (64, 8, 8),
]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_forward_layout(native, M, N, K):
    x, w = rnd(M, K, scale=0.5), rnd(N, K, scale=0.5, seed=1)
    bias = rnd(N, seed=2)
    got = native.linear(x, w, bias)
    ref = x.float() @ w.float().t() + bias.float()
    close(got, ref, rtol=2e-2, atol=2e-2 * (K ** 0.5) * 0.25)
    torch.cuda.synchronize()
    assert native.read_status(clear=False) == 0


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES[:6])
def test_gemm_dgrad_layout(native, M, N, K):
    dy, w = rnd(M, N, scale=0.5), rnd(N, K, scale=0.5, seed=1)
    got = native.linear_dgrad(dy, w)
    ref = dy.float() @ w.float()
    close(got, ref, rtol=2e-2, atol=2e-2 * (N ** 0.5) * 0.25)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES[:6])
def test_gemm_wgrad_layout_and_accumulate(native, M, N, K):
    dy, x = rnd(M, N, scale=0.5), rnd(M, K, scale=0.5, seed=1)
    got = native.linear_wgrad(dy, x)
    ref = dy.float().t() @ x.float()
    close(got, ref, rtol=2e-2, atol=2e-2 * (M ** 0.5) * 0.25)
    acc = torch.ones(N, K, dtype=torch.float32, device="cuda")
    native.linear_wgrad(dy, x, out=acc, accumulate=True)
    native.linear_wgrad(dy, x, out=acc, accumulate=True)
    close(acc, 1.0 + 2.0 * ref, rtol=2e-2, atol=4e-2 * (M ** 0.5) * 0.25)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H", [(37, 256), (128, 1600), (64, 4096), (16, 8192)])
def test_norms(native, dtype, rows, H):
    from jaxpp_b200.ops import core as ops

    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    x, w, b, dy = rnd(rows, H, dtype=dtype), rnd(H, dtype=dtype, seed=1), rnd(H, dtype=dtype, seed=2), rnd(rows, H, dtype=dtype, seed=3)
    y, rstd = native.rmsnorm(x, w, 1e-5)
    ry, rr = ops._rmsnorm_ref(x.float(), w.float(), 1e-5)
    close(y, ry, **tol)
    close(rstd, rr, rtol=1e-4, atol=1e-4)
    dx, dw = native.rmsnorm_bwd(dy, x, w, rstd)
    rdx, rdw = ops._rmsnorm_bwd_ref(dy.float(), x.float(), w.float(), rr)
    close(dx, rdx, **tol)
    close(dw, rdw, rtol=tol["rtol"], atol=tol["atol"] * rows ** 0.5)
    y, mean, rstd = native.layernorm(x, w, b, 1e-5)
    ry, rm, rr = ops._layernorm_ref(x.float(), w.float(), b.float(), 1e-5)
    close(y, ry, **tol)
    close(mean, rm, rtol=1e-4, atol=1e-4)
    dx, dw, db = native.layernorm_bwd(dy, x, w, mean, rstd)
    rdx, rdw, rdb = ops._layernorm_bwd_ref(dy.float(), x.float(), w.float(), rm, rr)
    close(dx, rdx, **tol)
    close(dw, rdw, rtol=tol["rtol"], atol=tol["atol"] * rows ** 0.5)
    close(db, rdb, rtol=tol["rtol"], atol=tol["atol"] * rows ** 0.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations_rope_colsum(native, dtype):
    from jaxpp_b200.ops import core as ops

    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    x, dy = rnd(33, 1024, dtype=dtype), rnd(33, 1024, dtype=dtype, seed=1)
    close(native.gelu(x), ops._gelu_ref(x.float()), **tol)
    close(native.gelu_bwd(dy, x), ops._gelu_bwd_ref(dy.float(), x.float()), **tol)
    gu, d2 = rnd(33, 2048, dtype=dtype, seed=2), rnd(33, 1024, dtype=dtype, seed=3)
    close(native.swiglu(gu), ops._swiglu_ref(gu.float()), **tol)
    close(native.swiglu_bwd(d2, gu), ops._swiglu_bwd_ref(d2.float(), gu.float()), **tol)
    close(native.colsum(x), x.float().sum(0), rtol=tol["rtol"], atol=tol["atol"] * 6)
    q = rnd(2, 16, 4, 128, dtype=dtype, seed=4)
    ang = torch.rand(16, 64, device="cuda") * 6.28
    cos, sin = ang.cos(), ang.sin()
    r = native.rope(q, cos, sin, False)
    close(r, ops._rope_ref(q.float(), cos, sin, False), **tol)
    close(native.rope(r, cos, sin, True), q, rtol=tol["rtol"] * 2, atol=tol["atol"] * 2)
    # fused split of a packed qkv projection (+ RoPE on q, k) and its transpose
    for hq, hkv, rope_on in ((4, 2, True), (3, 3, False)):
        packed = rnd(2, 16, hq + 2 * hkv, 128, dtype=dtype, seed=5)
        c, s_ = (cos, sin) if rope_on else (None, None)
        got = native.qkv_split(packed, c, s_, hq, hkv)
        ref = ops._qkv_split_ref(packed.float(), c, s_, hq, hkv)
        for g, r_ in zip(got, ref):
            assert g.is_contiguous()
            close(g, r_, **tol)
        merged = native.qkv_merge(*got, c, s_)
        close(merged, packed, rtol=tol["rtol"] * 2, atol=tol["atol"] * 2)  # merge inverts split
        close(merged, ops._qkv_merge_ref(*[g.float() for g in got], c, s_), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_backward_with_residual_add_rounds_like_two_kernels(native, dtype):
    """dx + add from one kernel must equal norm_bwd followed by a separate add bit for bit."""
    rows, H = 77, 1024
    x, dy, add = rnd(rows, H, dtype=dtype, seed=51), rnd(rows, H, dtype=dtype, seed=52), rnd(rows, H, dtype=dtype, seed=53)
    w, b = rnd(H, dtype=dtype, seed=54), rnd(H, dtype=dtype, seed=55)
    _, rstd = native.rmsnorm(x, w, 1e-5)
    dx, dw = native.rmsnorm_bwd(dy, x, w, rstd)
    dx2, dw2 = native.rmsnorm_bwd_add(dy, x, w, rstd, add)
    assert torch.equal(dx2, dx + add) and torch.equal(dw2, dw)
    _, mean, rstd = native.layernorm(x, w, b, 1e-5)
    dx, dw, db = native.layernorm_bwd(dy, x, w, mean, rstd)
    dx2, dw2, db2 = native.layernorm_bwd_add(dy, x, w, mean, rstd, add)
    assert torch.equal(dx2, dx + add) and torch.equal(dw2, dw) and torch.equal(db2, db)


def test_narrow_linear_like_a_router(native):
    """A linear layer with 4 outputs (a small router): the narrow operands of its backward GEMMs are re-pitched."""
    x, w, dy = rnd(300, 256, seed=41), rnd(4, 256, scale=0.2, seed=42), rnd(300, 4, seed=43)
    close(native.linear(x, w, None), x.float() @ w.float().t(), rtol=2e-2, atol=0.1)
    close(native.linear_dgrad(dy, w), dy.float() @ w.float(), rtol=2e-2, atol=0.05)
    close(native.linear_wgrad(dy, x), dy.float().t() @ x.float(), rtol=2e-2, atol=0.5)
    acc = torch.ones(4, 256, dtype=torch.float32, device="cuda")
    native.linear_wgrad(dy, x, out=acc, accumulate=True)
    close(acc, 1 + dy.float().t() @ x.float(), rtol=2e-2, atol=0.5)


@pytest.mark.parametrize("E,M,N,K", [(3, 192, 320, 256), (2, 200, 264, 128), (4, 64, 128, 64)])
def test_grouped_gemm_equal_groups(native, E, M, N, K):
    """One launch over all groups against per-group fp32 matmuls, in the three linear-layer layouts.  Group sizes
    that are not multiples of the tile make tiles straddle two groups: the masked rows / columns must not leak."""
    x, w = rnd(E, M, K, seed=31), rnd(E, N, K, scale=0.2, seed=32)
    dy = rnd(E, M, N, seed=33)
    close(native.linear_batched(x, w), torch.bmm(x.float(), w.float().transpose(1, 2)), rtol=2e-2, atol=2e-2 * K ** 0.5 * 0.2)
    if N % 64 == 0:
        close(native.linear_dgrad_batched(dy, w), torch.bmm(dy.float(), w.float()), rtol=2e-2, atol=2e-2 * N ** 0.5 * 0.2)
    else:
        close(native.linear_dgrad_batched(dy, w), torch.bmm(dy.float(), w.float()), rtol=2e-2, atol=2e-2 * N ** 0.5 * 0.2)
    ref_w = torch.bmm(dy.float().transpose(1, 2), x.float())
    close(native.linear_wgrad_batched(dy, x, torch.float32), ref_w, rtol=2e-2, atol=2e-2 * M ** 0.5)
    close(native.linear_wgrad_batched(dy, x), ref_w, rtol=2e-2, atol=3e-2 * M ** 0.5)


@pytest.mark.parametrize("E,seg,segs,N,K", [(3, 200, 2, 320, 256), (2, 384, 1, 512, 128), (4, 80, 4, 256, 64)])
def test_grouped_gemm_unequal_groups(native, E, seg, segs, N, K):
    from jaxpp_b200.utils import config

    with config.moe_skip_empty_slots.set(2):   # row counts used by all three GEMMs
        _grouped_gemm_unequal_groups(native, E, seg, segs, N, K)


def _grouped_gemm_unequal_groups(native, E, seg, segs, N, K):
    """Groups of different sizes inside equal-sized storage: each group's rows are ``segs`` segments of ``seg`` rows
    with a filled prefix (given in ``counts``) and zeros behind it.  Skipping what holds no data must not change any
    of the three products; entirely empty groups and segments, full ones and ones that end inside a tile are covered,
    and the output of skipped tiles must be written (zeros), not left as it was."""
    M = seg * segs
    if M % 64:
        M = None
    g = torch.Generator().manual_seed(7)
    counts = torch.randint(0, seg + 1, (E, segs), generator=g, dtype=torch.int32)
    counts[0, 0] = seg          # a full segment
    counts[-1] = 0              # a group without any data
    if E > 2:
        counts[1, -1] = 1       # a single row
    live = (torch.arange(seg)[None, None, :] < counts[:, :, None]).reshape(E, seg * segs, 1).cuda()
    counts = counts.cuda()
    rows = seg * segs
    x = rnd(E, rows, K, seed=51) * live
    dy = rnd(E, rows, N, seed=52) * live
    w = rnd(E, N, K, scale=0.2, seed=53)
    # outputs are fresh allocations: leave NaNs in the block that the caching allocator hands out next
    junk = torch.full((E, rows, max(N, K)), float("nan"), dtype=torch.bfloat16, device="cuda")
    del junk
    y = native.linear_batched(x, w, counts, seg)
    assert torch.isfinite(y.float()).all()
    close(y, torch.bmm(x.float(), w.float().transpose(1, 2)), rtol=2e-2, atol=2e-2 * K ** 0.5 * 0.2)
    junk = torch.full((E, rows, max(N, K)), float("nan"), dtype=torch.bfloat16, device="cuda")
    del junk
    dx = native.linear_dgrad_batched(dy, w, counts, seg)
    assert torch.isfinite(dx.float()).all()
    close(dx, torch.bmm(dy.float(), w.float()), rtol=2e-2, atol=2e-2 * N ** 0.5 * 0.2)
    if M is not None:
        ref_w = torch.bmm(dy.float().transpose(1, 2), x.float())
        junk = torch.full((E, N, K), float("nan"), dtype=torch.float32, device="cuda")
        del junk
        dw = native.linear_wgrad_batched(dy, x, torch.float32, counts, seg)
        assert torch.isfinite(dw).all()
        close(dw, ref_w, rtol=2e-2, atol=2e-2 * rows ** 0.5)
        assert dw[-1].abs().max().item() == 0.0      # the empty group's gradient is exactly zero
        close(native.linear_wgrad_batched(dy, x, None, counts, seg), ref_w, rtol=2e-2, atol=3e-2 * rows ** 0.5)
        # as a gradient sink: added onto an fp32 accumulator in the epilogue (empty groups leave it alone)
        from jaxpp_b200.ops import sink

        acc = torch.ones(E, N, K, dtype=torch.float32, device="cuda")
        got = sink.accumulate(torch.ops.b200.linear_wgrad_batched.default, acc, dy, x, torch.float32, counts, seg)
        assert got is acc
        close(acc, 1.0 + ref_w, rtol=2e-2, atol=2e-2 * rows ** 0.5)
        assert (acc[-1] == 1.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_kernel(native, dtype):
    from jaxpp_b200.parallel import moe
    import jaxpp_b200 as jp

    for T, E, k in ((1000, 8, 2), (77, 16, 4)):
        logits = rnd(T, E, dtype=dtype, seed=21)
        with jp.MpmdMesh.create({"mpmd": 1, "data": 1, "model": 1}, kind="cuda", multi_process=False):
            top_i, w, probs, hits = torch.ops.b200moe.router(logits, k)
        r_i, r_w, r_p, r_h = moe._route_ref(logits, k)
        close(probs, r_p, rtol=1e-4, atol=1e-6)
        assert torch.equal(top_i.sort(-1).values, r_i.sort(-1).values)
        close(w.sort(-1).values, r_w.sort(-1).values, rtol=1e-4, atol=1e-6)
        assert torch.equal(hits, r_h)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dropout_matches_counter_based_reference(native, dtype):
    from jaxpp_b200.ops import core as ops

    x = rnd(37, 129, dtype=dtype, seed=11)   # odd element count: the last Philox block is partial
    seed = torch.tensor(0x1234567812345, dtype=torch.int64, device="cuda")
    for p_drop, offset in ((0.1, 0), (0.5, 3), (0.0, 9)):
        got = native.dropout(x, p_drop, seed, offset)
        ref = ops._dropout_ref(x, p_drop, seed, offset)
        assert torch.equal(got == 0, ref == 0), "mask differs from the Philox reference"
        close(got, ref.float(), rtol=1e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-6)
    drop = (native.dropout(torch.ones(1 << 20, device="cuda"), 0.3, seed, 1) == 0).float().mean().item()
    assert abs(drop - 0.3) < 5e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_cross_entropy(native, dtype):
    from jaxpp_b200.ops import core as ops

    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    vocab, d = 1000, 256
    table = rnd(vocab, d, dtype=dtype)
    ids = torch.randint(0, vocab, (4, 77), device="cuda")
    assert torch.equal(native.embedding(ids, table), table[ids])
    dy = rnd(4, 77, d, dtype=dtype, seed=1)
    close(native.embedding_bwd(dy, ids, vocab), ops._emb_bwd_ref(dy.float(), ids, vocab), **tol)
    # the fp32 form (no cast pass) and the accumulating form that a microbatch loop's gradient sink uses
    ref32 = ops._emb_bwd_ref(dy.float(), ids, vocab, torch.float32)
    got32 = native.embedding_bwd(dy, ids, vocab, torch.float32)
    assert got32.dtype == torch.float32
    close(got32, ref32, rtol=1e-5, atol=1e-5)
    acc = torch.full_like(ref32, 0.5)
    assert native.embedding_bwd(dy, ids, vocab, out=acc, accumulate=True) is acc
    native.embedding_bwd(dy, ids, vocab, out=acc, accumulate=True)
    close(acc, 0.5 + 2 * ref32, rtol=1e-5, atol=1e-5)
    for V in (32000, 50257, 1000):
        logits = rnd(19, V, dtype=dtype, scale=3.0, seed=2)
        labels = torch.randint(0, V, (19,), device="cuda")
        loss, lse = native.cross_entropy(logits, labels)
        rl, rlse = ops._ce_ref(logits.float(), labels)
        close(loss, rl, rtol=1e-4, atol=1e-3)
        close(lse, rlse, rtol=1e-4, atol=1e-3)
        dl = torch.rand(19, device="cuda")
        got = native.cross_entropy_bwd(dl, logits, labels, lse)
        close(got, ops._ce_bwd_ref(dl, logits.float(), labels, rlse), rtol=tol["rtol"], atol=1e-3)


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_adamw(native, gdtype):
    from jaxpp_b200.ops import core as ops

    n = 100003
    p, g = rnd(n, dtype=torch.float32), rnd(n, dtype=gdtype, seed=1)
    m, v = rnd(n, dtype=torch.float32, scale=0.1, seed=2), rnd(n, dtype=torch.float32, scale=0.1, seed=3).abs()
    step = torch.tensor(3, device="cuda")
    args = (1e-3, 0.9, 0.95, 1e-8, 0.1, 0.5)
    got = native.adamw(p, g, m, v, step, *args, torch.bfloat16)
    ref = ops._adamw_ref(p, g, m, v, step, *args, torch.bfloat16)
    for a, b in zip(got[:3], ref[:3]):
        close(a, b, rtol=1e-5, atol=1e-6)
    close(got[3], ref[3], rtol=1e-2, atol=1e-2)


def test_ops_dispatch_to_native_and_autograd(native):
    """The b200:: ops route CUDA tensors to the native kernels and differentiate through them."""
    from jaxpp_b200.ops import core as ops

    x = rnd(256, 512).requires_grad_()
    w = rnd(1024, 512, scale=0.05, seed=1).requires_grad_()
    g = rnd(512, seed=2).requires_grad_()
    h = ops.rmsnorm(x, g, 1e-5)[0]
    y = ops.swiglu(ops.linear(h, w, None))
    y.float().pow(2).mean().backward()
    xr, wr, gr = (t.detach().float().requires_grad_() for t in (x, w, g))
    hr = ops._rmsnorm_ref(xr, gr, 1e-5)[0]
    yr = ops._swiglu_ref(hr @ wr.t())
    yr.pow(2).mean().backward()
    close(y, yr, rtol=3e-2, atol=3e-2)
    close(x.grad, xr.grad, rtol=5e-2, atol=2e-3)
    close(w.grad, wr.grad, rtol=5e-2, atol=2e-3)
    close(g.grad, gr.grad, rtol=5e-2, atol=5e-3)


ATTN_CASES = [
    # B, Sq, Sk, H, Hkv, D, causal
    (2, 256, 256, 4, 4, 64, True),
    (1, 512, 512, 4, 2, 128, True),
    (2, 384, 384, 2, 2, 128, False),
    (1, 200, 200, 2, 1, 64, True),   # ragged sequence: masks past the end of K and padded query rows
    (1, 1024, 1024, 8, 2, 128, True),
    # different query and key lengths: what ring attention's zigzag layout and any cached-key use call
    (1, 512, 256, 4, 2, 128, False),   # all queries against half as many keys
    (2, 256, 512, 4, 4, 64, False),    # half the queries against all keys
    (1, 256, 640, 4, 2, 128, True),    # causal with an offset: query i sees keys up to i + (Sk - Sq)
    (1, 200, 328, 2, 2, 64, True),     # the same, ragged
]


@pytest.mark.parametrize("B,Sq,Sk,H,Hkv,D,causal", ATTN_CASES)
def test_flash_attention_forward_backward(native, B, Sq, Sk, H, Hkv, D, causal):
    from jaxpp_b200.ops import attention as att
    from jaxpp_b200.ops import core as ops

    q, k, v = rnd(B, Sq, H, D, seed=1), rnd(B, Sk, Hkv, D, seed=2), rnd(B, Sk, Hkv, D, seed=3)
    do = rnd(B, Sq, H, D, seed=4)
    scale = D ** -0.5
    o, lse = att.attention_fwd(q, k, v, causal, scale)
    ro, rlse = ops._attn_ref(q.float(), k.float(), v.float(), causal, scale)
    close(o, ro, rtol=2e-2, atol=2e-2)
    close(lse, rlse, rtol=1e-3, atol=2e-3)
    dq, dk, dv = att.attention_bwd(do, q, k, v, o, lse, causal, scale)
    rdq, rdk, rdv = ops._attn_bwd_ref(do.float(), q.float(), k.float(), v.float(), ro, rlse, causal, scale)
    close(dq, rdq, rtol=3e-2, atol=3e-2)
    close(dk, rdk, rtol=3e-2, atol=3e-2 * (H // Hkv) ** 0.5)
    close(dv, rdv, rtol=3e-2, atol=3e-2 * (H // Hkv) ** 0.5)
    torch.cuda.synchronize()
    assert native.read_status(clear=False) == 0
