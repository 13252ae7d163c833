"""Multi-GPU worker (one process per GPU, NCCL): fused tensor-parallel kernels against their NCCL twins,
and the pipelined language-model step across GPUs.  Run under ``jaxpp_b200.launch``."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import jaxpp_b200 as jp  # noqa: E402
from jaxpp_b200.launch import distributed_main  # noqa: E402
from jaxpp_b200.ops import native  # noqa: E402
from jaxpp_b200.parallel import fused, tp  # noqa: E402
from jaxpp_b200.utils import config  # noqa: E402


def rnd(*shape, seed, scale=0.5):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def close(a, b, atol, what):
    torch.testing.assert_close(a.float(), b.float(), rtol=3e-2, atol=atol, msg=lambda m: f"{what}: {m}")


def scenario_fused_tp():
    n = dist.get_world_size()
    r = dist.get_rank()
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": 1, "model": n}, kind="cuda", multi_process=True)
    with mesh:
        for rep, (Ml, K, N) in enumerate([(256, 512, 768), (128 * 3, 1024, 264), (1024, 2048, 4096), (256, 512, 768)]):
            M = Ml * n
            x_shard, w = rnd(Ml, K, seed=10 + r + rep), rnd(N, K, seed=3 + rep, scale=0.1)
            bias = rnd(N, seed=5)
            with config.use_fused_collectives.set(False):
                ref = torch.ops.b200tp.ag_linear(x_shard, w, bias, "model")
            got = torch.ops.b200tp.ag_linear(x_shard, w, bias, "model")
            close(got, ref, 0.05, f"ag_linear {Ml}x{K}x{N}")
            # ... and against fp32 math on the gathered operand (not only against the twin, which shares the GEMM)
            parts = [torch.empty_like(x_shard) for _ in range(n)]
            dist.all_gather(parts, x_shard)
            x_all = torch.cat(parts).float()
            close(got, x_all @ w.float().t() + bias.float(), 0.02 * K ** 0.5 * 0.5 * 0.1 + 0.05, f"ag_linear vs fp32 {Ml}x{K}x{N}")
            # GEMM -> reduce-scatter
            x_full, w_row = rnd(M, K, seed=20 + r + rep), rnd(N, K, seed=30 + r + rep, scale=0.1)
            with config.use_fused_collectives.set(False):
                ref = torch.ops.b200tp.linear_rs(x_full, w_row, "model")
            got = torch.ops.b200tp.linear_rs(x_full, w_row, "model")
            close(got, ref, 0.08, f"linear_rs {M}x{K}x{N}")
            total = x_full.float() @ w_row.float().t()          # this rank's partial product in fp32 ...
            dist.all_reduce(total)                              # ... summed over the ranks
            close(got, total[r * Ml:(r + 1) * Ml], 0.02 * (n * K) ** 0.5 * 0.5 * 0.1 + 0.08, f"linear_rs vs fp32 {M}x{K}x{N}")
            # backward ops
            dy = rnd(M, N, seed=40 + r + rep)
            with config.use_fused_collectives.set(False):
                ref_dx = torch.ops.b200tp.dgrad_rs(dy, w, "model")
                ref_dw = torch.ops.b200tp.ag_wgrad(dy, x_shard, "model", torch.float32)
            close(torch.ops.b200tp.dgrad_rs(dy, w, "model"), ref_dx, 0.08, "dgrad_rs")
            got_dw = torch.ops.b200tp.ag_wgrad(dy, x_shard, "model", torch.float32)
            close(got_dw, ref_dw, 0.05 * (M ** 0.5) / 8, "ag_wgrad")
            dx32 = dy.float() @ w.float()
            dist.all_reduce(dx32)
            close(torch.ops.b200tp.dgrad_rs(dy, w, "model"), dx32[r * Ml:(r + 1) * Ml], 0.02 * (n * N) ** 0.5 * 0.5 * 0.1 + 0.08,
                  "dgrad_rs vs fp32")
            close(got_dw, dy.float().t() @ x_all, 0.02 * M ** 0.5 * 0.25 + 0.05, "ag_wgrad vs fp32")
            dy_shard = rnd(Ml, N, seed=50 + r + rep)
            with config.use_fused_collectives.set(False):
                ref_dx2, ref_full = torch.ops.b200tp.ag_dgrad(dy_shard, w, "model")
            got_dx2, got_full = torch.ops.b200tp.ag_dgrad(dy_shard, w, "model")
            close(got_dx2, ref_dx2, 0.08, "ag_dgrad dx")
            assert torch.equal(got_full, ref_full), "ag_dgrad gathered dy"
            close(got_dx2, got_full.float() @ w.float(), 0.02 * N ** 0.5 * 0.5 * 0.1 + 0.08, "ag_dgrad vs fp32")
        # all-reduce over peer memory (three calls: both buffer parities and a reuse)
        for rep, (numel, dt) in enumerate([(3 * 1024 * 1024 + 5, torch.float32), (2 * 1024 * 1024, torch.bfloat16),
                                           (1024 * 1024 + 3, torch.float32)]):
            g = torch.Generator(device="cuda").manual_seed(70 + r + rep)
            t = torch.randn(numel, generator=g, device="cuda").to(dt)
            ref = t.clone()
            dist.all_reduce(ref)
            got = fused.all_reduce(t, "model", 1.0)
            close(got, ref, 1e-5 if dt == torch.float32 else 0.05, f"all_reduce {numel} {dt}")
        torch.cuda.synchronize()
        assert native.read_status() == 0, "a fused kernel reported a time-out"
        assert fused.FALLBACKS[0] == 0, f"{fused.FALLBACKS[0]} fused calls fell back to NCCL"
        from jaxpp_b200.parallel import symm

        dist.barrier()
        assert symm.check_all_canaries(), "a kernel wrote outside a symmetric workspace"
        assert all(ws.buf.check_canaries() for ws in fused._AR_WS.values()), "all-reduce wrote outside its workspace"
    if r == 0:
        print("fused tensor-parallel kernels match their NCCL twins", flush=True)


def scenario_pp_gpu(schedule_name):
    """Pipeline ranks on separate GPUs with NCCL point-to-point transfers; the eager (sequential) step on
    this GPU with the same kernels is the oracle, so results must agree exactly."""
    from torch.utils import _pytree as pytree

    from helpers import make_mlp_step, mlp_params

    world = dist.get_world_size()
    sched = {"std": jp.Std1F1B(world), "interleaved": jp.Interleaved1F1B(2 * world, world), "zb": jp.ZeroBubble(world)}[schedule_name]
    mesh = jp.MpmdMesh.create({"mpmd": world, "data": 1, "model": 1}, kind="cuda", multi_process=True)
    dev = torch.device("cuda", torch.cuda.current_device())
    n_mb = 4
    params = pytree.tree_map(lambda t: t.to(dev), mlp_params(sched.num_stages, 64, dtype=torch.bfloat16))
    batch = torch.randn(n_mb, 32, 64, generator=torch.Generator().manual_seed(1)).to(dev, torch.bfloat16)
    step = make_mlp_step(sched.num_stages, sched, n_mb)
    ref = step(params, batch)
    f = jp.mpmd_jit_with_loop(step, mesh)
    got = f(params, batch)
    got2 = f(got[1], batch)
    ref2 = step(ref[1], batch)
    torch.cuda.synchronize()
    checked = 0
    for r_, g_ in ((ref, got), (ref2, got2)):
        for x, y in zip(pytree.tree_leaves(r_), pytree.tree_leaves(g_, is_leaf=lambda a: isinstance(a, jp.MpmdArray))):
            t = y.local_tensor()
            if t is not None:
                assert torch.equal(t, x), f"pipelined result differs from the eager step (max {(t.float() - x.float()).abs().max()})"
                checked += 1
    assert checked > 0 and native.read_status() == 0
    if dist.get_rank() == 0:
        print(f"pipeline over NCCL p2p ({schedule_name}) matches the eager step", flush=True)


def scenario_fused_moe():
    """Expert-parallel dispatch / combine as peer-memory kernels against the index-op + NCCL all-to-all path,
    forward and backward, several calls in a row (both buffer parities)."""
    from jaxpp_b200.parallel import moe

    n, r = dist.get_world_size(), dist.get_rank()
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind="cuda", multi_process=True)
    E, k, d = 4 * n, 2, 512
    with mesh:
        for rep, T in enumerate([256, 384, 256]):
            capacity = (int(-(-T * k * 1.0 // E)) + 7) // 8 * 8
            g = torch.Generator(device="cuda").manual_seed(100 + r + 7 * rep)
            x0 = (torch.randn(T, d, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
            top_i = torch.stack([torch.randperm(E, generator=g, device="cuda")[:k] for _ in range(T)])
            w0 = torch.rand(T * k, generator=g, device="cuda")
            dest, keep = moe.slots_for(top_i, E, capacity)
            res = {}
            for fused_on in (False, True):
                with config.use_fused_collectives.set(fused_on):
                    x = x0.clone().requires_grad_(True)
                    w = w0.clone().requires_grad_(True)
                    buf = torch.ops.b200moe.dispatch_a2a(x, dest, None, E, capacity, k, "data")
                    y = (buf.float() * 1.5 + 0.25).to(torch.bfloat16)
                    out, picked = torch.ops.b200moe.combine_a2a(y, dest, w, E, capacity, k, "data", True)
                    loss = (out.float() * torch.linspace(-1, 1, d, device="cuda")).sum()
                    gx, gw = torch.autograd.grad(loss, [x, w])
                    scaled = torch.ops.b200moe.dispatch_a2a(x0, dest, w0, E, capacity, k, "data")
                    res[fused_on] = (buf.detach(), out.detach(), picked.detach(), gx, gw, scaled)
            names = ["dispatch", "combine out", "picked", "grad x", "grad weights", "scaled dispatch"]
            for name, a, b in zip(names, res[False], res[True]):
                if name in ("dispatch", "picked", "scaled dispatch"):
                    assert torch.equal(a, b), f"{name}: fused differs from the all-to-all path (T={T})"
                else:
                    close(b, a, 0.05, f"{name} (T={T})")
        torch.cuda.synchronize()
        assert native.read_status() == 0, "a fused kernel reported a time-out"
        from jaxpp_b200.parallel import fused_moe

        dist.barrier()
        assert all(ws.buf.check_canaries() for ws in fused_moe._WS.values()), "dispatch / combine wrote outside the buffer"
    if r == 0:
        print("fused MoE dispatch / combine match the NCCL all-to-all path", flush=True)


def scenario_p2p_native():
    """The C-ABI NCCL point-to-point backend on its own: several dtypes (fp8 included) in one grouped transfer, both
    directions, twice (the second transfer reuses the communicators and streams)."""
    from jaxpp_b200.runtime.p2p_native import NcclP2P

    r = dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    p2p = NcclP2P([(0, 1), (1, 0)], dev)

    def payload(seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        base = torch.randn(3, 1000, generator=g, device="cuda")
        return [base.clone(), base.to(torch.bfloat16), base.to(torch.float8_e4m3fn), (base * 100).to(torch.int64),
                torch.empty(0, device="cuda"), base[:, :7].contiguous()]

    for rep in range(2):
        mine, theirs = payload(10 * rep + r), payload(10 * rep + (1 - r))
        bufs = [torch.empty_like(t) for t in theirs]
        ready = torch.cuda.Event()
        ready.record()
        done_r = p2p.recv(1 - r, bufs, ready)
        done_s = p2p.send(1 - r, mine, ready)
        torch.cuda.current_stream().wait_event(done_r)
        torch.cuda.current_stream().wait_event(done_s)
        torch.cuda.synchronize()
        for got, want in zip(bufs, theirs):
            assert got.dtype == want.dtype and torch.equal(got.view(torch.uint8), want.view(torch.uint8)), want.dtype
    p2p.close()
    if r == 0:
        print("native NCCL p2p backend: fp32 / bf16 / fp8 / int64 payloads round-trip", flush=True)


def scenario_moe_train_gpu():
    """A Mixtral-style train step with experts sharded over two GPUs (the data axis doubles as the expert axis):
    router kernel, fused dispatch / combine over peer memory and grouped expert GEMMs, against the same step with the
    index-op + NCCL all-to-all path.  Tight capacity, so some picks are dropped."""
    from torch.utils import _pytree as pytree

    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf

    n = dist.get_world_size()
    sched = jp.Std1F1B(1)
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind="cuda", multi_process=True)
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = tf.ModelConfig("mixtral", vocab=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn=512, seq=128, n_stages=1,
                         tp=1, dtype=torch.bfloat16, n_experts=4, top_k=2, capacity_factor=1.25, ep=n, aux_coef=0.01)
    hyper = lt.Hyper(lr=1e-3, inplace_update=False)
    g = torch.Generator().manual_seed(11 + dist.get_rank())      # every data-parallel rank has its own sequences
    tokens = torch.randint(0, 512, (2, 2, 128), generator=g).to(dev)
    labels = torch.randint(0, 512, (2, 2, 128), generator=g).to(dev)
    results = {}
    for fused_on in (False, True):
        with config.use_fused_collectives.set(fused_on):
            state = lt.init_state(cfg, sched, dev, my_rank=0, tp_rank=0, seed=0)
            f = jp.mpmd_jit_with_loop(lt.make_train_step(cfg, sched, hyper, dp_axis="data", dp=n), mesh)
            state, losses = f(state, tokens, labels)
            state, losses2 = f(state, tokens, labels)
            torch.cuda.synchronize()
            results[fused_on] = (state, losses, losses2)
    assert native.read_status() == 0, "a fused kernel reported a time-out"
    from jaxpp_b200.parallel import fused_moe

    assert fused_moe._WS, "the expert exchange did not go through the peer-memory kernels"
    is_arr = lambda a: isinstance(a, jp.MpmdArray)
    checked = 0
    for a, b in zip(pytree.tree_leaves(results[False], is_leaf=is_arr), pytree.tree_leaves(results[True], is_leaf=is_arr)):
        ta, tb = a.local_tensor(), b.local_tensor()
        if ta is None or not ta.is_floating_point():
            continue
        torch.testing.assert_close(tb.float(), ta.float(), rtol=5e-2, atol=5e-3)
        checked += 1
    assert checked > 0
    if dist.get_rank() == 0:
        print("Mixtral-style step with expert parallelism: fused MoE kernels match the NCCL path", flush=True)


def scenario_zero_gpu():
    """Optimizer state sharded over two data-parallel GPUs.  (1) The peer-memory reduce-scatter and all-gather
    kernels against NCCL for fp32 / bf16 and sizes that need padding.  (2) A GPT-2-style train step whose master
    weights and moments are 1/dp slices against the same step with whole state and all-reduced gradients."""
    from torch.utils import _pytree as pytree

    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf
    from jaxpp_b200.parallel import zero

    n, r = dist.get_world_size(), dist.get_rank()
    sched = jp.Std1F1B(1)
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind="cuda", multi_process=True)
    dev = torch.device("cuda", torch.cuda.current_device())
    with mesh:
        for dtype, numel in ((torch.float32, 1 << 20), (torch.float32, 1000003), (torch.bfloat16, 3 * 1000 * 1000 + 5)):
            x = (torch.randn(numel, generator=torch.Generator().manual_seed(7 + r)) * 0.5).to(dev).to(dtype)
            s = zero.shard_numel(numel, n)
            want = torch.zeros(s * n, dtype=torch.float32, device=dev)
            want[:numel] = x.float()
            dist.all_reduce(want)
            want = want * 0.25
            got = fused.reduce_scatter_flat(x, "data", 0.25)
            assert got.shape == (s,) and got.dtype == dtype
            # fp32: exact with two ranks; with more the order of the additions differs from NCCL's by an ulp
            tol = (0 if n == 2 else 1e-6) if dtype == torch.float32 else 2e-2
            torch.testing.assert_close(got.float(), want[r * s:(r + 1) * s], rtol=tol, atol=tol)
            # the op picks the same kernel
            torch.testing.assert_close(zero.reduce_scatter_flat(x, "data", 0.25), got, rtol=0, atol=0)
            full = fused.all_gather_flat(got, "data")
            parts = [torch.empty_like(got) for _ in range(n)]
            dist.all_gather(parts, got)
            assert torch.equal(full, torch.cat(parts))
            assert torch.equal(zero.all_gather_flat(got, "data", numel), torch.cat(parts)[:numel])
        torch.cuda.synchronize()
        assert native.read_status() == 0, "a peer-memory collective reported a time-out"
        for ws in fused._AR_WS.values():
            ws.buf.check_canaries()

    cfg = tf.ModelConfig("gpt2", vocab=2048, d_model=512, n_layers=2, n_heads=8, n_kv_heads=8, ffn=2048, seq=128, n_stages=1,
                         tp=1, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(3 + r)
    tokens = torch.randint(0, 2048, (2, 2, 128), generator=g).to(dev)
    labels = torch.randint(0, 2048, (2, 2, 128), generator=g).to(dev)
    results = {}
    for sharded in (False, True):
        hyper = lt.Hyper(lr=1e-3, inplace_update=False, shard_optimizer=sharded)
        state = lt.init_state(cfg, sched, dev, my_rank=0, tp_rank=0, seed=0)
        if sharded:
            state = lt.shard_state_for_dp(cfg, state, n, r)
        f = jp.mpmd_jit_with_loop(lt.make_train_step(cfg, sched, hyper, dp_axis="data", dp=n), mesh)
        state, losses = f(state, tokens, labels)
        state, losses2 = f(state, tokens, labels)
        torch.cuda.synchronize()
        results[sharded] = (state, losses, losses2)
    assert native.read_status() == 0, "a fused kernel reported a time-out"
    is_arr = lambda a: isinstance(a, jp.MpmdArray)
    whole, shard = results[False], results[True]
    for a, b in zip(pytree.tree_leaves((whole[0]["params"], whole[1], whole[2]), is_leaf=is_arr),
                    pytree.tree_leaves((shard[0]["params"], shard[1], shard[2]), is_leaf=is_arr)):
        torch.testing.assert_close(b.local_tensor().float(), a.local_tensor().float(), rtol=1e-2, atol=2e-3)
    for key in ("master", "m"):
        for a, b in zip(pytree.tree_leaves(whole[0][key], is_leaf=is_arr), pytree.tree_leaves(shard[0][key], is_leaf=is_arr)):
            want = zero.local_shard(a.local_tensor(), n, r)
            assert b.local_tensor().shape == want.shape
            torch.testing.assert_close(b.local_tensor(), want, rtol=1e-2, atol=2e-3 if key == "master" else 1e-4)
    if r == 0:
        print("sharded optimizer state: peer-memory reduce-scatter / all-gather match NCCL; train step matches", flush=True)


def scenario_ring_attention_gpu():
    """Context parallelism on GPUs: the native flash-attention kernels per block, NCCL point-to-point for the ring;
    forward and gradients against the native kernel on the whole sequence (bf16, grouped-query heads)."""
    from jaxpp_b200.ops import core as ops
    from jaxpp_b200.parallel import context

    n, r = dist.get_world_size(), dist.get_rank()
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind="cuda", multi_process=True)
    B, S, H, Hkv, D = 2, 512 * n, 8, 2, 128
    q, k, v, do = (rnd(B, S, h, D, seed=10 + i) for i, h in enumerate((H, Hkv, Hkv, H)))   # same on every rank
    scale = D ** -0.5
    chunk = lambda t: t[:, r * S // n:(r + 1) * S // n].contiguous()
    with mesh:
        for causal in (False, True):
            want, lse = ops.attention(q, k, v, causal, scale)
            dq, dk, dv = ops.attention_bwd(do, q, k, v, want, lse, causal, scale)
            ql, kl, vl = (chunk(t).requires_grad_() for t in (q, k, v))
            got = context.ring_attention(ql, kl, vl, causal, scale, "data")
            got.backward(chunk(do))
            torch.cuda.synchronize()
            close(got.detach(), chunk(want), 2e-2, f"ring attention forward causal={causal}")
            close(ql.grad, chunk(dq), 3e-2, f"ring attention dq causal={causal}")
            close(kl.grad, chunk(dk), 3e-2, f"ring attention dk causal={causal}")
            close(vl.grad, chunk(dv), 3e-2, f"ring attention dv causal={causal}")
    assert native.read_status() == 0
    if r == 0:
        print("ring attention on GPUs matches the single-GPU kernels", flush=True)


def scenario_pp_tied_gpu():
    """Tied input / output embeddings on two pipeline GPUs: the two ranks' gradient contributions are summed by a
    cross-stage all-reduce, which for a tensor this large runs as the one-kernel all-reduce over peer memory;
    the same step with NCCL collectives is the oracle."""
    from torch.utils import _pytree as pytree

    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf

    sched = jp.Std1F1B(2)
    mesh = jp.MpmdMesh.create({"mpmd": 2, "data": 1, "model": 1}, kind="cuda", multi_process=True)
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = tf.ModelConfig("llama", vocab=2048, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn=512, seq=128,
                         n_stages=2, tp=1, dtype=torch.bfloat16, tie_embeddings=True)
    hyper = lt.Hyper(lr=1e-3, inplace_update=False)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, 2048, (4, 2, 128), generator=g).to(dev)
    labels = torch.randint(0, 2048, (4, 2, 128), generator=g).to(dev)
    results = {}
    for fused_on in (False, True):
        with config.use_fused_collectives.set(fused_on):
            state = lt.init_state(cfg, sched, dev, my_rank=mesh.my_mpmd_axis_index, tp_rank=0, seed=0)
            f = jp.mpmd_jit_with_loop(lt.make_train_step(cfg, sched, hyper), mesh)
            state, losses = f(state, tokens, labels)
            torch.cuda.synchronize()
            results[fused_on] = (state, losses)
    assert native.read_status() == 0
    assert fused._AR_WS, "the cross-stage all-reduce did not go through the peer-memory kernel"
    is_arr = lambda a: isinstance(a, jp.MpmdArray)
    checked = 0
    for a, b in zip(pytree.tree_leaves(results[False], is_leaf=is_arr), pytree.tree_leaves(results[True], is_leaf=is_arr)):
        ta, tb = a.local_tensor(), b.local_tensor()
        if ta is None or not ta.is_floating_point():
            continue
        torch.testing.assert_close(tb.float(), ta.float(), rtol=2e-2, atol=2e-3)
        checked += 1
    assert checked > 0
    if dist.get_rank() == 0:
        print("tied embeddings: cross-stage all-reduce over peer memory matches NCCL", flush=True)


def scenario_pp_tp_gpu(pp, tp, schedule_name):
    """Pipeline x tensor parallel Llama-style step on pp*tp GPUs (bf16, native kernels): the fused
    compute+collective kernels against the same step with NCCL collectives, two steps each."""
    from torch.utils import _pytree as pytree

    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf

    n_stages = {"std": pp, "interleaved": 2 * pp}[schedule_name]
    sched = jp.Std1F1B(pp) if schedule_name == "std" else jp.Interleaved1F1B(n_stages, pp)
    mesh = jp.MpmdMesh.create({"mpmd": pp, "data": 1, "model": tp}, kind="cuda", multi_process=True)
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = tf.ModelConfig("llama", vocab=512, d_model=256, n_layers=n_stages, n_heads=4, n_kv_heads=2, ffn=512, seq=128,
                         n_stages=n_stages, tp=tp, dtype=torch.bfloat16)
    hyper = lt.Hyper(lr=1e-3, inplace_update=False)
    n_mb = 2 * n_stages
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, 512, (n_mb, 2 * tp, 128), generator=g).to(dev)
    labels = torch.randint(0, 512, (n_mb, 2 * tp, 128), generator=g).to(dev)
    me_pp, me_tp = mesh.my_mpmd_axis_index, mesh.axis_index("model")
    results = {}
    for fused_on in (False, True):
        with config.use_fused_collectives.set(fused_on):
            state = lt.init_state(cfg, sched, dev, my_rank=me_pp, tp_rank=me_tp, seed=0)
            f = jp.mpmd_jit_with_loop(lt.make_train_step(cfg, sched, hyper), mesh)
            state, losses1 = f(state, tokens, labels)
            state, losses2 = f(state, tokens, labels)
            torch.cuda.synchronize()
            results[fused_on] = (state, losses1, losses2)
    assert native.read_status() == 0, "a fused kernel reported a time-out"
    assert fused.FALLBACKS[0] == 0, f"{fused.FALLBACKS[0]} fused calls fell back to NCCL"
    is_arr = lambda a: isinstance(a, jp.MpmdArray)
    checked = 0
    for a, b in zip(pytree.tree_leaves(results[False], is_leaf=is_arr), pytree.tree_leaves(results[True], is_leaf=is_arr)):
        ta, tb = a.local_tensor(), b.local_tensor()
        if ta is None:
            continue
        if ta.dtype in (torch.int32, torch.int64):
            assert torch.equal(ta, tb)
        else:
            torch.testing.assert_close(tb.float(), ta.float(), rtol=5e-2, atol=5e-3)
        checked += 1
    assert checked > 0
    if dist.get_rank() == 0:
        print(f"pp{pp} x tp{tp} ({schedule_name}): fused collectives match NCCL through two steps", flush=True)


def scenario_dp_overlap():
    """Data-parallel gradient collectives issued from the last microbatch's backward tasks on the side stream (all-reduce,
    and reduce-scatter with sharded optimizer state) against the same step with the collectives after the loop: the
    same peer-memory kernels on the same operands, so the new states must be identical bit for bit."""
    from torch.utils import _pytree as pytree

    from jaxpp_b200.compiler.program import RunTask
    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf

    n, r = dist.get_world_size(), dist.get_rank()
    sched = jp.Std1F1B(1)
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind="cuda", multi_process=True)
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = tf.ModelConfig("gpt2", vocab=2048, d_model=1024, n_layers=2, n_heads=16, n_kv_heads=16, ffn=4096, seq=128, n_stages=1,
                         tp=1, dtype=torch.bfloat16)     # weight matrices of 2-8 MiB: above the peer-memory threshold
    g = torch.Generator().manual_seed(3 + r)
    tokens = torch.randint(0, 2048, (4, 2, 128), generator=g).to(dev)
    labels = torch.randint(0, 2048, (4, 2, 128), generator=g).to(dev)
    is_arr = lambda a: isinstance(a, jp.MpmdArray)
    for sharded in (False, True):
        results = {}
        for overlap in (False, True):
            with config.overlap_grad_reduce.set(overlap):
                hyper = lt.Hyper(lr=1e-3, inplace_update=False, shard_optimizer=sharded)
                state = lt.init_state(cfg, sched, dev, my_rank=0, tp_rank=0, seed=0)
                if sharded:
                    state = lt.shard_state_for_dp(cfg, state, n, r)
                f = jp.mpmd_jit_with_loop(lt.make_train_step(cfg, sched, hyper, dp_axis="data", dp=n), mesh)
                hooks = sum(len(i.hooks) for i in f.lower(state, tokens, labels).program.instrs if isinstance(i, RunTask))
                assert (hooks >= 8) == overlap, f"overlap={overlap}: {hooks} gradient collectives hooked into backward tasks"
                state, losses = f(state, tokens, labels)
                state, losses2 = f(state, tokens, labels)
                torch.cuda.synchronize()
                results[overlap] = (state, losses, losses2)
        assert native.read_status() == 0, "a peer-memory collective reported a time-out"
        for a, b in zip(pytree.tree_leaves(results[False], is_leaf=is_arr), pytree.tree_leaves(results[True], is_leaf=is_arr)):
            assert torch.equal(a.local_tensor(), b.local_tensor()), f"sharded={sharded}: overlapped gradient reduction differs"
    from jaxpp_b200.parallel import symm

    dist.barrier()
    assert symm.check_all_canaries()
    assert any(isinstance(k, tuple) and k and k[-1] == "side" for k in fused._AR_WS), "no collective ran on the side stream"
    if r == 0:
        print("gradient collectives overlapped with the backward pass match the after-loop form bit for bit", flush=True)


def scenario_vocab_parallel_gpu():
    """Output projection split by vocabulary rows over two tensor-parallel GPUs (sharded logits, combined log-sum-exps)
    against the replicated head on the same two GPUs, and the first-step loss against ln(vocab)-scale expectations."""
    from torch.utils import _pytree as pytree

    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf

    n = dist.get_world_size()
    sched = jp.Std1F1B(1)
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": 1, "model": n}, kind="cuda", multi_process=True)
    dev = torch.device("cuda", torch.cuda.current_device())
    me_tp = mesh.axis_index("model")
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, 1024, (2, 2, 128), generator=g).to(dev)
    labels = torch.randint(0, 1024, (2, 2, 128), generator=g).to(dev)
    losses = {}
    params = {}
    for vp in (False, True):
        cfg = tf.ModelConfig("llama", vocab=1024, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn=512, seq=128, n_stages=1,
                             tp=n, dtype=torch.bfloat16, vocab_parallel=vp)
        state = lt.init_state(cfg, sched, dev, my_rank=0, tp_rank=me_tp, seed=0)
        if vp:   # the same matrix as the replicated head: this rank's rows
            full = params[False]
            rows = full.shape[0] // n
            for key in ("params", "master"):
                state[key]["lm_head"] = full[me_tp * rows:(me_tp + 1) * rows].to(state[key]["lm_head"].dtype).clone()
        else:
            params[False] = state["master"]["lm_head"].clone()
        f = jp.mpmd_jit_with_loop(lt.make_train_step(cfg, sched, lt.Hyper(lr=1e-3, inplace_update=False)), mesh)
        new_state, l1 = f(state, tokens, labels)
        torch.cuda.synchronize()
        t = l1.local_tensor().float()
        dist.all_reduce(t)
        losses[vp] = t / n
        params[("head", vp)] = new_state["master"]["lm_head"].local_tensor()
    assert native.read_status() == 0
    torch.testing.assert_close(losses[True], losses[False], rtol=2e-2, atol=2e-2)
    rows = params[("head", False)].shape[0] // n
    torch.testing.assert_close(params[("head", True)], params[("head", False)][me_tp * rows:(me_tp + 1) * rows], rtol=0, atol=2.5e-3)
    if dist.get_rank() == 0:
        print("vocabulary-parallel head and cross entropy match the replicated head", flush=True)


def scenario_ring_attention_zigzag_gpu():
    """The zigzag sequence layout of ring attention on GPUs (pieces r and 2n-1-r per rank; calls the flash-attention
    kernels with different query and key lengths) against the single-GPU kernels on the whole sequence."""
    from jaxpp_b200.ops import core as ops
    from jaxpp_b200.parallel import context

    n, r = dist.get_world_size(), dist.get_rank()
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind="cuda", multi_process=True)
    B, S, H, Hkv, D = 2, 512 * n, 8, 2, 128
    q, k, v, do = (rnd(B, S, h, D, seed=10 + i) for i, h in enumerate((H, Hkv, Hkv, H)))
    scale = D ** -0.5
    with mesh:
        chunk = lambda t: context.local_sequence_slice(t, "data", 1, "zigzag").contiguous()
        want, lse = ops.attention(q, k, v, True, scale)
        dq, dk, dv = ops.attention_bwd(do, q, k, v, want, lse, True, scale)
        ql, kl, vl = (chunk(t).requires_grad_() for t in (q, k, v))
        got = context.ring_attention(ql, kl, vl, True, scale, "data", "zigzag")
        got.backward(chunk(do))
        torch.cuda.synchronize()
        close(got.detach(), chunk(want), 2e-2, "zigzag ring attention forward")
        close(ql.grad, chunk(dq), 3e-2, "zigzag ring attention dq")
        close(kl.grad, chunk(dk), 3e-2, "zigzag ring attention dk")
        close(vl.grad, chunk(dv), 3e-2, "zigzag ring attention dv")
    assert native.read_status() == 0
    if r == 0:
        print("zigzag ring attention on GPUs matches the single-GPU kernels", flush=True)


SCENARIOS = {
    "dp_overlap": scenario_dp_overlap,
    "vocab_parallel": scenario_vocab_parallel_gpu,
    "ring_attention_zigzag": scenario_ring_attention_zigzag_gpu,
    "fused_tp": scenario_fused_tp,
    "fused_moe": scenario_fused_moe,
    "pp_tied": scenario_pp_tied_gpu,
    "moe_train": scenario_moe_train_gpu,
    "zero": scenario_zero_gpu,
    "ring_attention": scenario_ring_attention_gpu,
    "p2p_native": scenario_p2p_native,
    "pp2_tp2_std": lambda: scenario_pp_tp_gpu(2, 2, "std"),
    "pp2_tp2_interleaved": lambda: scenario_pp_tp_gpu(2, 2, "interleaved"),
    "pp_std": lambda: scenario_pp_gpu("std"),
    "pp_interleaved": lambda: scenario_pp_gpu("interleaved"),
    "pp_zb": lambda: scenario_pp_gpu("zb"),
}

if __name__ == "__main__":
    distributed_main(SCENARIOS[sys.argv[1]], backend="nccl")
