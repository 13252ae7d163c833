"""Worker for the multi-process tests: ``python mp_worker.py <scenario>`` under ``jaxpp_b200.launch``.

Each scenario runs on every rank, computes the un-pipelined / un-sharded oracle locally where it can, and
exits non-zero on a mismatch.
"""
import os
import sys

import torch
import torch.distributed as dist
from torch.utils import _pytree as pytree

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import jaxpp_b200 as jp  # noqa: E402
from jaxpp_b200.launch import distributed_main  # noqa: E402
from jaxpp_b200.models import lm_trainer as lt  # noqa: E402
from jaxpp_b200.models import transformer as tf  # noqa: E402

from helpers import make_mlp_step, mlp_params  # noqa: E402


def device():
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def check_tree(ref, got, rtol, atol, what):
    a = pytree.tree_leaves(ref)
    b = pytree.tree_leaves(got, is_leaf=lambda x: isinstance(x, jp.MpmdArray))
    assert len(a) == len(b), what
    checked = 0
    for x, y in zip(a, b):
        t = y.local_tensor() if isinstance(y, jp.MpmdArray) else y
        if t is None:
            continue
        torch.testing.assert_close(t.cpu().float(), x.cpu().float(), rtol=rtol, atol=atol, msg=lambda m: f"{what}: {m}")
        checked += 1
    assert checked > 0, f"{what}: nothing was addressable on rank {dist.get_rank()}"


def scenario_pp(schedule, n_mb):
    """Pure pipeline parallelism: one process per stage rank, point-to-point transfers between them."""
    world = dist.get_world_size()
    mesh = jp.MpmdMesh.create({"mpmd": world, "data": 1, "model": 1}, kind=device().type, multi_process=True)
    params = mlp_params(schedule.num_stages, 16)
    batch = torch.randn(n_mb, 4, 16, generator=torch.Generator().manual_seed(1))
    step = make_mlp_step(schedule.num_stages, schedule, n_mb)
    ref = step(params, batch)
    dev = device()
    to = lambda t: pytree.tree_map(lambda x: x.to(dev), t)
    f = jp.mpmd_jit_with_loop(step, mesh)
    got = f(to(params), to(batch))
    exact = dev.type == "cpu"
    check_tree(ref, got, 0 if exact else 1e-5, 0 if exact else 1e-6, "pp step 1")
    me = mesh.my_mpmd_axis_index
    owner_last = schedule.get_mpmd_idx(schedule.num_stages - 1)
    assert got[0].is_partially_addressable == (me == owner_last)
    # feed the distributed result back in for a second step
    ref2 = step(ref[1], batch)
    got2 = f(got[1], to(batch))
    check_tree(ref2, got2, 0 if exact else 1e-5, 0 if exact else 1e-6, "pp step 2")


def scenario_stack():
    """cross_mpmd_stack of values that live on different pipeline ranks: one all-gather over the owners, with the
    ranks owning different numbers of operands (3 stages' statistics on 2 ranks)."""
    from jaxpp_b200.ops import core as ops

    world = dist.get_world_size()
    sched = jp.Interleaved1F1B(3 * world, world) if world > 1 else jp.Std1F1B(1)
    n_stages = sched.num_stages
    mesh = jp.MpmdMesh.create({"mpmd": world, "data": 1, "model": 1}, kind=device().type, multi_process=True)
    params = mlp_params(n_stages, 16)
    batch = torch.randn(4, 4, 16, generator=torch.Generator().manual_seed(1))
    inner = make_mlp_step(n_stages, sched, 4)

    def step(params, batch):
        loss, new = inner(params, batch)
        # per-layer statistics of the new weights: layers 0, 2, 4 (rank 0) and layer 1 (rank 1), stacked in this order
        picks = [0, 2, 1, 4] if n_stages >= 5 else list(range(n_stages))
        stats = jp.cross_mpmd_stack([new[i]["w1"].pow(2).sum(0) for i in picks], axis=0)
        return loss, new, stats

    ref = step(params, batch)
    dev = device()
    to = lambda t: pytree.tree_map(lambda x: x.to(dev), t)
    got = jp.mpmd_jit_with_loop(step, mesh)(to(params), to(batch))
    exact = dev.type == "cpu"
    check_tree(ref, got, 0 if exact else 1e-5, 0 if exact else 1e-6, "stack")
    assert got[2].is_partially_addressable and tuple(got[2].shape) == tuple(ref[2].shape)


def scenario_pp_tp(pp, tp, schedule):
    """Pipeline x tensor parallel language model against the un-sharded single-process step."""
    mesh = jp.MpmdMesh.create({"mpmd": pp, "data": 1, "model": tp}, kind=device().type, multi_process=True)
    dev = device()
    base = dict(vocab=250, d_model=64, n_layers=4, n_heads=4, n_kv_heads=2, ffn=128, seq=32, dtype=torch.float32,
                vocab_parallel=bool(os.environ.get("TEST_VOCAB_PARALLEL")))
    cfg1 = tf.ModelConfig("llama", n_stages=schedule.num_stages, tp=1, **base)
    cfgt = tf.ModelConfig("llama", n_stages=schedule.num_stages, tp=tp, **base)
    hyper = lt.Hyper(lr=1e-2, inplace_update=False, clip_grad_norm=float(os.environ["TEST_CLIP"]) if os.environ.get("TEST_CLIP") else None)
    n_mb = 4
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, 250, (n_mb, 2, 32), generator=g)
    labels = torch.randint(0, 250, (n_mb, 2, 32), generator=g)
    # oracle: plain eager step on the full model
    state1 = lt.init_state(cfg1, schedule, "cpu")
    ref_state, ref_losses = lt.make_train_step(cfg1, schedule, hyper)(state1, tokens, labels)
    # sharded state of this process: its pipeline rank's groups, its tensor-parallel shard
    me_pp, me_tp = mesh.my_mpmd_axis_index, mesh.axis_index("model")
    owners = lt.owner_ranks(cfgt, schedule)

    def local_view(tree, shard: bool):
        out = {}
        for key in ("params", "master", "m", "v"):
            full = tree[key]
            sharded = tf.shard_params_for_tp(cfg1, full, tp, me_tp) if shard else full
            sel = {"layers": {}}
            for name, layer in sharded["layers"].items():
                mine = owners[int(name)] == me_pp
                sel["layers"][name] = {k: (v.to(dev) if mine else jp.ShapeDtypeStruct(tuple(v.shape), v.dtype))
                                       for k, v in layer.items()}
            for k, v in sharded.items():
                if k == "layers":
                    continue
                grp = "embed" if k in ("embed", "pos") else "head"
                sel[k] = v.to(dev) if owners[grp] == me_pp else jp.ShapeDtypeStruct(tuple(v.shape), v.dtype)
            out[key] = sel
        out["step"] = tree["step"].to(dev)
        return out

    state_local = local_view(state1, shard=True)
    step = lt.make_train_step(cfgt, schedule, hyper)
    f = jp.mpmd_jit_with_loop(step, mesh)
    got_state, got_losses = f(state_local, tokens.to(dev), labels.to(dev))
    # compare: shard the oracle's result the same way
    ref_local = local_view(ref_state, shard=True)
    for key in ("params", "master", "m", "v"):
        a = pytree.tree_leaves(ref_local[key], is_leaf=lambda x: isinstance(x, jp.ShapeDtypeStruct))
        b = pytree.tree_leaves(got_state[key], is_leaf=lambda x: isinstance(x, jp.MpmdArray))
        assert len(a) == len(b)
        n = 0
        for x, y in zip(a, b):
            t = y.local_tensor()
            if isinstance(x, jp.ShapeDtypeStruct):
                assert t is None, "a non-owner rank holds data"
                continue
            if key == "m":  # linear in the (clipped) gradient: a wrong clip coefficient shows here
                torch.testing.assert_close(t.cpu(), x.cpu(), rtol=2e-3, atol=1e-7)
            else:
                torch.testing.assert_close(t.cpu(), x.cpu(), rtol=2e-3, atol=5e-4)  # Adam amplifies reassociation noise where g ~ 0
            n += 1
        assert n > 0
    lt_ = got_losses.local_tensor()
    if lt_ is not None:
        # each tensor-parallel rank reports the mean loss of its own token slice
        per_tok = ref_losses  # [n_mb] mean over all tokens
        both = lt_.clone()
        dist.all_reduce(both, group=mesh.axis_group("model"))
        torch.testing.assert_close((both / tp).cpu(), per_tok, rtol=1e-4, atol=1e-5)
    elif tp > 1 and mesh.axis_group("model") is not None:
        pass


def scenario_dp_ep(family, shard_optimizer=False):
    """2 pipeline ranks x 2 data-parallel ranks.  ``gpt2``: plain data parallelism (gradients all-reduced over
    the data axis); ``mixtral``: the data axis doubles as the expert-parallel axis (experts sharded, tokens
    exchanged with all-to-all).  ``shard_optimizer``: master weights and Adam moments are 1/dp slices per rank,
    gradients are reduce-scattered and parameters all-gathered.  Oracle: the un-sharded step on the concatenated
    batch."""
    pp, dp = 2, 2
    mesh = jp.MpmdMesh.create({"mpmd": pp, "data": dp, "model": 1}, kind=device().type, multi_process=True)
    dev = device()
    sched = jp.Std1F1B(2)
    base = dict(vocab=250, d_model=32, n_layers=2, n_heads=2, n_kv_heads=2, ffn=64, seq=16, dtype=torch.float32, n_stages=2)
    # aux_coef 0: the load-balancing statistics are per rank by design, so only the task loss is comparable
    moe = dict(n_experts=4, top_k=2, capacity_factor=8.0, aux_coef=0.0) if family == "mixtral" else {}
    context_parallel = family.startswith("llama_cp")   # the data axis carries chunks of every sequence instead of sequences
    cp_layout = "zigzag" if family.endswith("zigzag") else "contiguous"
    family = "llama" if context_parallel else family
    cfg1 = tf.ModelConfig(family, **base, **moe)
    cfgd = tf.ModelConfig(family, **base, **moe, ep=dp if family == "mixtral" else 1, cp=dp if context_parallel else 1, cp_layout=cp_layout,
                          recompute=bool(os.environ.get("TEST_RECOMPUTE")))
    hyper = lt.Hyper(lr=1e-2, inplace_update=False, clip_grad_norm=float(os.environ["TEST_CLIP"]) if os.environ.get("TEST_CLIP") else None)
    n_mb, mb = 2, 4
    g = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, 250, (n_mb, mb, 16), generator=g)
    labels = torch.randint(0, 250, (n_mb, mb, 16), generator=g)
    state1 = lt.init_state(cfg1, sched, "cpu")
    ref_state, ref_losses = lt.make_train_step(cfg1, sched, hyper)(state1, tokens, labels)
    me_pp, me_dp = mesh.my_mpmd_axis_index, mesh.axis_index("data")
    owners = lt.owner_ranks(cfgd, sched)
    e_local = cfgd.n_experts // cfgd.ep if family == "mixtral" else 0

    def shard_experts(k, v):
        if family == "mixtral" and k in ("e_up", "e_down"):
            return v[me_dp * e_local:(me_dp + 1) * e_local]
        return v

    def local_view(tree):
        out = {}
        for key in ("params", "master", "m", "v"):
            full = tree[key]
            sel = {"layers": {}}
            for name, layer in full["layers"].items():
                mine = owners[int(name)] == me_pp
                sel["layers"][name] = {}
                for k, v in layer.items():
                    v = shard_experts(k, v)
                    sel["layers"][name][k] = v.to(dev) if mine else jp.ShapeDtypeStruct(tuple(v.shape), v.dtype)
            for k, v in full.items():
                if k == "layers":
                    continue
                grp = "embed" if k in ("embed", "pos") else "head"
                sel[k] = v.to(dev) if owners[grp] == me_pp else jp.ShapeDtypeStruct(tuple(v.shape), v.dtype)
            out[key] = sel
        out["step"] = tree["step"].to(dev)
        return out

    if shard_optimizer:
        import dataclasses

        whole_view = local_view
        local_view = lambda tree: lt.shard_state_for_dp(cfgd, whole_view(tree), dp, me_dp)
        hyper_d = dataclasses.replace(hyper, shard_optimizer=True)
    else:
        hyper_d = hyper
    step = (lt.make_train_step(cfgd, sched, hyper_d) if context_parallel
            else lt.make_train_step(cfgd, sched, hyper_d, dp_axis="data", dp=dp))
    f = jp.mpmd_jit_with_loop(step, mesh)
    if context_parallel:
        if cp_layout == "zigzag":
            pc = 16 // (2 * dp)
            cut = lambda t: torch.cat([t[:, :, me_dp * pc:(me_dp + 1) * pc],
                                       t[:, :, (2 * dp - 1 - me_dp) * pc:(2 * dp - me_dp) * pc]], dim=2)
        else:
            part = 16 // dp  # this rank's chunk of every sequence
            cut = lambda t: t[:, :, me_dp * part:(me_dp + 1) * part]
        tok_l, lab_l = cut(tokens).contiguous().to(dev), cut(labels).contiguous().to(dev)
    else:
        half = mb // dp  # this data-parallel rank's sequences of every microbatch
        tok_l = tokens[:, me_dp * half:(me_dp + 1) * half].contiguous().to(dev)
        lab_l = labels[:, me_dp * half:(me_dp + 1) * half].contiguous().to(dev)
    got_state, got_losses = f(local_view(state1), tok_l, lab_l)
    if not context_parallel and os.environ.get("TEST_OVERLAP"):
        # the gradient collectives issued from inside the last microbatch's backward tasks against the same step with
        # the collectives after the loop: same kernels on the same operands, so bit for bit
        from jaxpp_b200.compiler.program import RunTask
        from jaxpp_b200.utils import config

        prog = f.lower(local_view(state1), tok_l, lab_l).program
        n_hooks = sum(len(i.hooks) for i in prog.instrs if isinstance(i, RunTask))
        assert n_hooks >= 6, f"only {n_hooks} gradient collectives were moved into the backward pass"
        with config.overlap_grad_reduce.set(False):
            f_after = jp.mpmd_jit_with_loop(step, mesh)
            prog_after = f_after.lower(local_view(state1), tok_l, lab_l).program
            assert not any(i.hooks for i in prog_after.instrs if isinstance(i, RunTask))
            after_state, after_losses = f_after(local_view(state1), tok_l, lab_l)
        a = pytree.tree_leaves(after_state, is_leaf=lambda x: isinstance(x, jp.MpmdArray))
        b = pytree.tree_leaves(got_state, is_leaf=lambda x: isinstance(x, jp.MpmdArray))
        compared = 0
        for x, y in zip(a, b):
            tx, ty = x.local_tensor(), y.local_tensor()
            assert (tx is None) == (ty is None)
            if tx is not None:
                assert torch.equal(tx, ty), "overlapped and after-loop gradient reduction differ"
                compared += 1
        assert compared > 0
    ref_local = local_view(ref_state)
    # with capacity-based routing the per-rank capacity differs from the single-rank run only if tokens are dropped;
    # the generous capacity factor above keeps every token, so results agree up to reassociation
    n = 0
    for key in ("params", "m"):
        a = pytree.tree_leaves(ref_local[key], is_leaf=lambda x: isinstance(x, jp.ShapeDtypeStruct))
        b = pytree.tree_leaves(got_state[key], is_leaf=lambda x: isinstance(x, jp.MpmdArray))
        for x, y in zip(a, b):
            t = y.local_tensor()
            if isinstance(x, jp.ShapeDtypeStruct):
                assert t is None
                continue
            if key == "m":  # first moment = (1 - beta1) * gradient: linear in the gradient
                torch.testing.assert_close(t.cpu(), x.cpu(), rtol=1e-3, atol=1e-7)
            else:  # Adam's first step is +-lr per element: reassociation noise flips the sign where g ~ 0
                bad = ((t.cpu() - x.cpu()).abs() > 5e-4).float().mean().item()
                assert bad < 0.01, f"{bad:.3%} of a parameter tensor differs"
            n += 1
    assert n > 0


def scenario_ring_attention():
    """Context parallelism: every rank holds one contiguous chunk of the sequence; forward output and the gradients of
    q, k, v against full attention on the whole sequence (grouped-query heads, causal and not), eagerly and through a
    captured pipelined step."""
    from jaxpp_b200.ops import core as ops
    from jaxpp_b200.parallel import context

    n, r = dist.get_world_size(), dist.get_rank()
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind=device().type, multi_process=True)
    dev = device()
    B, S, H, Hkv, D = 2, 8 * n, 4, 2, 16
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(B, S, h, D, generator=g) for h in (H, Hkv, Hkv))
    do = torch.randn(B, S, H, D, generator=g)
    scale = D ** -0.5
    piece = S // (2 * n)
    chunks = {"contiguous": lambda t: t[:, r * S // n:(r + 1) * S // n].contiguous().to(dev),
              "zigzag": lambda t: torch.cat([t[:, r * piece:(r + 1) * piece],
                                             t[:, (2 * n - 1 - r) * piece:(2 * n - r) * piece]], dim=1).contiguous().to(dev)}
    chunk = chunks["contiguous"]
    with mesh:
        for causal, layout in ((False, "contiguous"), (True, "contiguous"), (True, "zigzag"), (False, "zigzag")):
            chunk = chunks[layout]
            qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
            want, _ = ops.attention(qf, kf, vf, causal, scale)
            want.backward(do)
            ql, kl, vl = (chunk(t).requires_grad_() for t in (q, k, v))
            got = context.ring_attention(ql, kl, vl, causal, scale, "data", layout)
            got.backward(chunk(do))
            torch.testing.assert_close(got.detach().cpu(), chunk(want.detach()).cpu(), rtol=1e-5, atol=1e-5)
            for name, a, b in (("dq", ql.grad, qf.grad), ("dk", kl.grad, kf.grad), ("dv", vl.grad, vf.grad)):
                torch.testing.assert_close(a.cpu(), chunk(b).cpu(), rtol=1e-4, atol=1e-5, msg=lambda m: f"{name} causal={causal}: {m}")
            assert torch.equal(context.local_sequence_slice(q.to(dev), "data", 1, layout), chunk(q))
        chunk = chunks["contiguous"]

    # inside a compiled step (one pipeline rank, the data axis as the context axis)
    w = (torch.randn(H * D, H * D, generator=g) * 0.1).to(dev)

    def step(w, q, k, v):
        def body(mb):
            qb, kb, vb = mb

            def loss_fn(w):
                o = context.ring_attention(qb, kb, vb, True, scale, "data")
                y = jp.mark_stage_end(ops.linear(o.reshape(-1, H * D), w, None))
                return (y ** 2).sum()

            return jp.value_and_grad(loss_fn)(w)

        return jp.treduce(body, (q, k, v), schedule=jp.Std1F1B(1))

    stack = lambda t: torch.stack([chunk(t), chunk(t) * 0.5])
    losses, gw = jp.mpmd_jit_with_loop(step, mesh)(w, stack(q), stack(k), stack(v))
    with mesh:
        ref_losses, ref_gw = step(w, stack(q), stack(k), stack(v))
    torch.testing.assert_close(losses.local_tensor().cpu(), ref_losses.cpu(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(gw.local_tensor().cpu(), ref_gw.cpu(), rtol=1e-5, atol=1e-5)
    full_o, _ = ops.attention(q, k, v, True, scale)
    want_loss = (ops.linear(chunk(full_o).reshape(-1, H * D), w, None) ** 2).sum()
    torch.testing.assert_close(losses.local_tensor()[0].cpu(), want_loss.cpu(), rtol=1e-4, atol=1e-4)


def scenario_reshard():
    """SPMD -> MPMD -> SPMD round trip of arrays with several partition specs."""
    from jaxpp_b200.array import DistArray, MpmdSharding, mpmd_to_spmd_reshard, spmd_to_mpmd_reshard
    from jaxpp_b200.mesh import NamedSharding, P

    world = dist.get_world_size()
    assert world == 4
    mesh = jp.MpmdMesh.create({"mpmd": 2, "data": 1, "model": 2}, kind=device().type, multi_process=True)
    g = torch.Generator().manual_seed(0)
    xs = [torch.randn(8, 12, generator=g), torch.randn(4, 6, generator=g), torch.arange(16.0).view(16, 1)]
    src_specs = [P(("mpmd", "model"), None), P(None, "model"), P("mpmd", None)]
    dst = [MpmdSharding(mesh, {1}, P(None, "model")), MpmdSharding(mesh, {0, 1}, P("model", None)),
           MpmdSharding(mesh, set(), P())]
    me = mesh.my_device
    arrays = [DistArray.from_global(x, NamedSharding(mesh.jax_mesh, s), devices=[me]) for x, s in zip(xs, src_specs)]
    moved = spmd_to_mpmd_reshard(mesh, arrays, dst, threshold=1, donate=False)
    my_pp = mesh.my_mpmd_axis_index
    assert moved[0].mpmd_idxs == (1,) and moved[0].is_partially_addressable == (my_pp == 1)
    assert moved[1].mpmd_idxs == (0, 1) and moved[1].is_partially_addressable
    assert moved[2].mpmd_idxs == (0,)  # empty mesh_ids parks the array on rank 0
    if my_pp == 1:
        want = xs[0][NamedSharding(mesh.unstack[1], P(None, "model")).device_index(me, xs[0].shape)]
        assert torch.equal(moved[0].local_tensor().cpu(), want)
    want1 = xs[1][NamedSharding(mesh.unstack[my_pp], P("model", None)).device_index(me, xs[1].shape)]
    assert torch.equal(moved[1].local_tensor().cpu(), want1)
    back = mpmd_to_spmd_reshard(mesh, moved, [NamedSharding(mesh.jax_mesh, s) for s in src_specs])
    for x, s, arr in zip(xs, src_specs, back):
        want = x[NamedSharding(mesh.jax_mesh, s).device_index(me, x.shape)]
        assert torch.equal(arr.shards[me].cpu(), want), s


SCENARIOS = {
    "pp_std1f1b": lambda: scenario_pp(jp.Std1F1B(dist.get_world_size()), 4),
    "pp_interleaved": lambda: scenario_pp(jp.Interleaved1F1B(2 * dist.get_world_size(), dist.get_world_size()), 4),
    "pp_zb": lambda: scenario_pp(jp.ZeroBubble(dist.get_world_size()), 4),
    "pp_dualpipev": lambda: scenario_pp(jp.DualPipeV(2 * dist.get_world_size(), dist.get_world_size()), 4),
    "pp2_tp2": lambda: scenario_pp_tp(2, 2, jp.Interleaved1F1B(4, 2)),
    "tp2": lambda: scenario_pp_tp(1, 2, jp.Std1F1B(1)),
    "reshard": scenario_reshard,
    "stack": scenario_stack,
    "ring_attention": scenario_ring_attention,
    "pp2_dp2_gpt2": lambda: scenario_dp_ep("gpt2"),
    "pp2_ep2_mixtral": lambda: scenario_dp_ep("mixtral"),
    "pp2_cp2_llama": lambda: scenario_dp_ep("llama_cp"),
    "pp2_cp2_llama_zigzag": lambda: scenario_dp_ep("llama_cp_zigzag"),
    "pp2_dp2_gpt2_zero": lambda: scenario_dp_ep("gpt2", shard_optimizer=True),
    "pp2_ep2_mixtral_zero": lambda: scenario_dp_ep("mixtral", shard_optimizer=True),
}

if __name__ == "__main__":
    name = sys.argv[1]
    distributed_main(SCENARIOS[name])
