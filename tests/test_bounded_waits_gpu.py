"""Every device-side wait of the native library is bounded: when it runs out, the kernel returns and the status word
says why.  These tests make waits run out on purpose, in the only form that leaves the GPU healthy: a flag (or an
mbarrier) that nobody raises and a wait budget of a few milliseconds.  Nothing here traps, faults or spins forever.

The "peer" of the fused kernels is emulated on one GPU: the call descriptor of rank 0 of a 2-rank group whose second
rank's buffers are ordinary local allocations that no kernel ever signals from.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

BUDGET_MS = 20.0
GUARD = 256
PATTERN = 0xA5


@pytest.fixture()
def native():
    from jaxpp_b200.ops import native as n

    n.load()
    torch.cuda.synchronize()
    n.read_status()                      # start clean
    n.set_wait_budget_ms(BUDGET_MS)
    yield n
    torch.cuda.synchronize()
    n.set_wait_budget_ms(4000.0)         # the library's default, for whatever test runs next in this process
    n.read_status()


def _guarded(nbytes: int):
    """A zeroed byte buffer with a patterned guard band on either side; returns (whole, usable pointer)."""
    whole = torch.zeros(nbytes + 2 * GUARD, dtype=torch.uint8, device="cuda")
    whole[:GUARD] = PATTERN
    whole[GUARD + nbytes:] = PATTERN
    return whole, whole.data_ptr() + GUARD


def _canaries_ok(whole, nbytes) -> bool:
    return bool((whole[:GUARD] == PATTERN).all() and (whole[GUARD + nbytes:] == PATTERN).all())


def test_mbarrier_wait_runs_out_and_reports(native):
    lib = native.load()
    lib.jpb_selftest_mbar_timeout.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    assert lib.jpb_selftest_mbar_timeout(out.data_ptr(), native._stream()) == 0
    torch.cuda.synchronize()                       # returns: the kernel did not hang
    timed_out, spent_ns = out.tolist()
    assert timed_out == 1
    assert 2 * BUDGET_MS * 1e6 <= spent_ns < 100 * BUDGET_MS * 1e6   # waits inside a CTA get twice the budget
    assert native.read_status() == 1               # JPB_ERR_WAIT_TIMEOUT
    # the context is healthy: an ordinary kernel runs and is correct
    x = torch.randn(256, 128, device="cuda").bfloat16()
    w = torch.randn(64, 128, device="cuda").bfloat16()
    torch.testing.assert_close(native.linear(x, w, None).float(), x.float() @ w.float().t(), rtol=2e-2, atol=0.2)
    torch.cuda.synchronize()
    assert native.read_status() == 0


def _fake_two_rank_comm_desc(symm, ctrl_bytes, g_bytes, r_bytes):
    """Descriptor of rank 0 of 2 whose 'peer' buffers are local memory nobody signals from."""
    total = ctrl_bytes + g_bytes + r_bytes
    bufs = [_guarded(total) for _ in range(2)]
    d = symm.JpbCommDesc()
    d.n_ranks, d.rank, d.epoch = 2, 0, 1
    d.max_ctas = 0
    for q in range(2):
        base = bufs[q][1]
        d.ctrl[q] = base
        d.g[q] = base + ctrl_bytes
        d.r[q] = base + ctrl_bytes + g_bytes
    return d, bufs, total


@pytest.mark.parametrize("kind", ["gather", "scatter"])
def test_fused_gemm_gives_up_on_a_silent_peer(native, kind):
    from jaxpp_b200.parallel import fused, symm

    lib = fused._lib()
    lib.jpb_comm_ctrl_bytes.restype = ctypes.c_longlong
    ctrl = (lib.jpb_comm_ctrl_bytes() + 1023) // 1024 * 1024
    M, N, K = 512, 256, 128                        # 2 ranks x 2 row tiles
    x_shard = torch.randn(M // 2, K, device="cuda").bfloat16()
    x_full = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    desc, bufs, total = _fake_two_rank_comm_desc(symm, ctrl, M * K * 2, M * N * 2)
    if kind == "gather":                           # all-gather -> GEMM: waits for the peer's chunk flags
        desc.gather, desc.scatter = fused.GATHER_ROWS, 0
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        fused._launch(x_shard, w, out, None, M, N, K, K, K, False, False, False, desc)
    else:                                          # GEMM -> reduce-scatter: waits for the peer's tile flags
        desc.gather, desc.scatter = 0, 1
        out = torch.empty(M // 2, N, dtype=torch.bfloat16, device="cuda")
        fused._launch(x_full, w, out, None, M, N, K, K, K, False, False, False, desc)
    torch.cuda.synchronize()                       # the kernel returned
    assert native.read_status() == 3               # JPB_ERR_PEER_TIMEOUT
    for whole, _ in bufs:
        assert _canaries_ok(whole, total)
    with pytest.raises(native.KernelStatusError):  # what a training loop sees
        fused._launch(x_full, w, out, None, M, N, K, K, K, False, False, False, desc) if kind == "scatter" else \
            fused._launch(x_shard, w, out, None, M, N, K, K, K, False, False, False, desc)
        native.raise_on_status("test step")
    # the next ordinary launch works
    torch.testing.assert_close(native.linear(x_full, w, None).float(), x_full.float() @ w.float().t(), rtol=2e-2, atol=0.3)
    torch.cuda.synchronize()
    assert native.read_status() == 0


def test_peer_memory_all_reduce_gives_up_on_a_silent_peer(native):
    from jaxpp_b200.parallel import fused

    lib = fused._lib()
    lib.jpb_allreduce.argtypes = [ctypes.POINTER(fused._AllReduceDesc), ctypes.c_void_p]
    n = 1 << 16
    ctrl, slot = 1024, n * 4
    bufs = [_guarded(ctrl + slot) for _ in range(2)]
    d = fused._AllReduceDesc()
    d.n_ranks, d.rank, d.epoch, d.dtype, d.mode = 2, 0, 1, 0, 0
    d.n, d.scale, d.grid = n, 1.0, 8
    d.counter_target = 8
    for q in range(2):
        d.ctrl[q] = bufs[q][1]
        d.x[q] = bufs[q][1] + ctrl
    out = torch.full((n,), 7.0, device="cuda")
    d.out = out.data_ptr()
    assert lib.jpb_allreduce(ctypes.byref(d), native._stream()) == 0
    torch.cuda.synchronize()
    assert native.read_status() == 3
    assert bool((out == 7.0).all())                # gave up before writing anything
    for whole, _ in bufs:
        assert _canaries_ok(whole, ctrl + slot)


def test_router_with_non_finite_logits_keeps_indices_in_range(native):
    from jaxpp_b200.parallel import moe  # noqa: F401  (registers the op)

    T, E, k = 64, 8, 2
    logits = torch.randn(T, E, device="cuda")
    logits[5] = float("nan")
    logits[17, 3] = float("nan")
    top_i, weights, probs, hits = torch.ops.b200moe.router(logits, k)
    torch.cuda.synchronize()
    assert int(top_i.min()) >= 0 and int(top_i.max()) < E
    assert top_i[5].tolist() == [0, 1] and top_i[17].tolist() == [0, 1]   # the lowest experts not yet taken
    assert native.read_status() == 2               # JPB_ERR_BAD_ARGUMENT: reported, not silently accepted
    ok = torch.ones(T, dtype=torch.bool, device="cuda")
    ok[5] = ok[17] = False
    ref = torch.softmax(logits[ok].float(), -1)
    torch.testing.assert_close(probs[ok], ref, rtol=1e-4, atol=1e-5)
    assert bool((top_i[ok] == ref.topk(k, dim=-1).indices).all())
