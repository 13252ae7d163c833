"""Compiler equivalence: the scheduled multi-rank program, interpreted in one process, must give
bit-identical results to the plain sequential step — for every schedule family."""
import pytest
import torch
from torch.utils import _pytree as pytree

import jaxpp_b200 as jp
from jaxpp_b200.compiler.program import AllReduce, RunTask, Transfer
from jaxpp_b200.compiler.verify import verify_program
from jaxpp_b200.ops import core as ops
from jaxpp_b200.utils import config

from helpers import assert_trees_equal, leaves, local, make_mlp_step, mlp_forward, mlp_params

CASES = [
    # (mpmd_dim, schedule, n_mubatches)
    (2, jp.Std1F1B(2), 4),
    (4, jp.Std1F1B(4), 8),
    (3, jp.Eager1F1B(3), 5),
    (2, jp.GPipe(2), 3),
    (2, jp.Interleaved1F1B(4, 2), 4),
    (4, jp.Interleaved1F1B(8, 4), 8),
    (2, jp.Interleaved1F1B(4, 2, fuse_steady_state=True), 4),
    (2, jp.KimiK2(4, 2), 4),
    (4, jp.ZeroBubble(4), 6),
    (2, jp.DualPipeV(4, 2), 4),
    (4, jp.DualPipeV(8, 4), 10),
]


def cpu_mesh(pp):
    return jp.MpmdMesh.create({"mpmd": pp, "data": 1, "model": 1}, kind="cpu", multi_process=False)


@pytest.mark.parametrize("pp,schedule,n_mb", CASES, ids=lambda c: str(c).replace(" ", ""))
def test_scheduled_program_is_bit_exact(pp, schedule, n_mb):
    n_layers = schedule.num_stages
    params = mlp_params(n_layers, 16)
    batch = torch.randn(n_mb, 4, 16, generator=torch.Generator().manual_seed(1))
    step = make_mlp_step(schedule.num_stages, schedule, n_mb)
    ref = step(params, batch)
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(pp))
    got = f(params, batch)
    assert_trees_equal(ref, got, exact=True)
    compiled = f.lower(params, batch)
    verify_program(compiled.program)
    # losses live on the rank of the last stage, each layer's params where its stage runs
    assert got[0].mpmd_idxs == (schedule.get_mpmd_idx(schedule.num_stages - 1),)
    for layer, p in enumerate(got[1]):
        assert p["w1"].mpmd_idxs == (schedule.get_mpmd_idx(layer),)


@pytest.mark.parametrize("pp,schedule,n_mb", [(8, jp.Interleaved1F1B(48, 8), 64), (8, jp.DualPipeV(16, 8), 18)],
                         ids=["interleaved48x64", "dualpipev16x18"])
def test_big_shapes_compile(pp, schedule, n_mb):
    params = mlp_params(schedule.num_stages, 8)
    batch = torch.randn(n_mb, 2, 8)
    step = make_mlp_step(schedule.num_stages, schedule, n_mb)
    compiled = jp.mpmd_jit_with_loop(step, cpu_mesh(pp)).lower(params, batch)
    stats = compiled.program.stats()
    assert stats["n_tasks"] > schedule.num_stages * n_mb
    verify_program(compiled.program)
    # structurally identical stages share executables
    assert stats["n_executables"] < 64


def test_fusion_flag_unpacks_fused_tasks():
    sched = jp.Interleaved1F1B(4, 2)
    params, batch = mlp_params(4, 8), torch.randn(4, 2, 8)
    step = make_mlp_step(4, sched, 4)
    fused = jp.mpmd_jit_with_loop(step, cpu_mesh(2)).lower(params, batch).program
    assert any(i.name.startswith("fused_") for i in fused.instrs if isinstance(i, RunTask))
    with config.disable_schedule_task_fusion.set(True):
        plain = jp.mpmd_jit_with_loop(step, cpu_mesh(2)).lower(params, batch).program
    assert not any(i.name.startswith("fused_") for i in plain.instrs if isinstance(i, RunTask))
    assert sum(isinstance(i, RunTask) for i in plain.instrs) > sum(isinstance(i, RunTask) for i in fused.instrs)


def test_zero_bubble_split_separates_weight_grads():
    sched = jp.ZeroBubble(2)
    params, batch = mlp_params(2, 8), torch.randn(2, 2, 8)
    prog = jp.mpmd_jit_with_loop(make_mlp_step(2, sched, 2), cpu_mesh(2)).lower(params, batch).program
    by_name = {i.name.split("__")[0]: i for i in prog.instrs if isinstance(i, RunTask)}
    assert "bwdA_1" in by_name and "bwdW_1" in by_name and "bwdW_0" not in by_name
    ops_of = lambda name: " ".join(str(t) for t in by_name[name].code.targets)
    assert "linear_wgrad" in ops_of("bwdW_1") and "linear_wgrad" not in ops_of("bwdA_1")
    assert "linear_dgrad" in ops_of("bwdA_1") and "linear_dgrad" not in ops_of("bwdW_1")


def test_shared_weight_gradients_use_cross_rank_all_reduce():
    """A weight used by the first and the last stage: each rank accumulates its own partial gradient
    and the partials are summed once after the loop."""
    sched = jp.Std1F1B(2)
    n_mb = 4
    g = torch.Generator().manual_seed(3)
    params = {"emb": torch.randn(8, 8, generator=g) * 0.3, "mid": torch.randn(8, 8, generator=g) * 0.3}
    batch = torch.randn(n_mb, 4, 8, generator=g)

    def step(params, batch):
        def body(mb):
            def loss_fn(p):
                x = ops.linear(mb, p["emb"], None)
                x = jp.mark_stage_end(ops.gelu(x))
                x = ops.linear(x, p["mid"], None)
                x = ops.linear(x, p["emb"], None)  # tied weight on the last stage
                x = jp.mark_stage_end(x)
                return (x ** 2).mean() / n_mb

            return jp.value_and_grad(loss_fn)(params)

        loss, grads = jp.treduce(body, batch, schedule=sched)
        return loss, pytree.tree_map(lambda p, gr: p - 0.5 * gr, params, grads)

    ref = step(params, batch)
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
    got = f(params, batch)
    prog = f.lower(params, batch).program
    assert sum(isinstance(i, AllReduce) for i in prog.instrs) == 2  # one instruction per participant
    # no weight-sized transfer inside the loop: only the [4, 8] activations and their gradients move
    assert all(prog.values[v].shape == (4, 8) for i in prog.instrs if isinstance(i, Transfer) for v in i.vids)
    assert got[1]["emb"].mpmd_idxs == (0, 1) and got[1]["mid"].mpmd_idxs == (1,)
    assert_trees_equal(ref, got, exact=False, rtol=1e-6, atol=1e-7)
    verify_program(prog)


def test_after_loop_requires_explicit_collective():
    sched = jp.Std1F1B(2)
    params, batch = mlp_params(2, 8), torch.randn(2, 2, 8)

    def step(params, batch):
        loss, grads = make_inner(params, batch)
        norm = sum((g ** 2).sum() for g in pytree.tree_leaves(grads))  # mixes ranks without a collective
        return loss, norm

    def make_inner(params, batch):
        def body(mb):
            def loss_fn(p):
                return ((mlp_forward(p, mb, 2) - mb) ** 2).mean()

            return jp.value_and_grad(loss_fn)(params)

        return jp.treduce(body, batch, schedule=sched)

    with pytest.raises(AssertionError, match="After loop computation is not replicateable"):
        jp.mpmd_jit_with_loop(step, cpu_mesh(2)).lower(params, batch)

    def step_ok(params, batch):
        loss, grads = make_inner(params, batch)
        per_stage = [sum((g ** 2).sum() for g in pytree.tree_leaves(layer)) for layer in grads]
        norm = jp.cross_mpmd_all_reduce(*per_stage).sqrt()
        stacked = jp.cross_mpmd_stack(per_stage)
        return loss, norm, stacked

    ref = step_ok(params, batch)
    got = jp.mpmd_jit_with_loop(step_ok, cpu_mesh(2))(params, batch)
    assert got[1].mpmd_idxs == (0, 1) and got[2].mpmd_idxs == (0, 1)
    assert_trees_equal(ref, got, exact=False)


def test_replicated_scalars_and_passthrough():
    """Values with no placement constraint (a step counter) are computed on every rank; inputs
    returned unchanged stay exact."""
    sched = jp.Std1F1B(2)
    params, batch = mlp_params(2, 8), torch.randn(2, 2, 8)
    inner = make_mlp_step(2, sched, 2)

    def step(params, batch, count, extra):
        loss, new = inner(params, batch)
        return loss, new, count + 1, extra

    count, extra = torch.tensor(7), torch.arange(3.0)
    out = jp.mpmd_jit_with_loop(step, cpu_mesh(2))(params, batch, count, extra)
    assert out[2].mpmd_idxs == (0, 1) and int(out[2]) == 8
    assert torch.equal(local(out[3]), extra)


def test_forward_only_pipeline_by_yield():
    params = mlp_params(4, 8)
    x = torch.randn(3, 8)

    def infer(params, x):
        return mlp_forward(params, x, 4).sum(-1)

    ref = infer(params, x)
    f = jp.mpmd_jit_by_yield(infer, cpu_mesh(2))
    got = f(params, x)
    assert torch.equal(local(got), ref)
    prog = f.lower(params, x).program
    ranks = [i.rank for i in prog.instrs if isinstance(i, RunTask)]
    assert ranks == [0, 1, 0, 1]  # stage s runs on rank s % mpmd_dim
    verify_program(prog)


def test_treduce_i_and_ops():
    sched = jp.Std1F1B(2)
    params = mlp_params(2, 8)
    batch = torch.randn(3, 2, 8)

    def step(params, batch):
        def body(i):
            mb = jp.take(batch, i)

            def loss_fn(p):
                out = mlp_forward(p, mb, 2)
                return ((out - mb) ** 2).mean(), out.detach().abs().amax()

            (loss, peak), grads = jp.value_and_grad(loss_fn, has_aux=True)(params)
            return loss, grads, peak

        return jp.treduce_i(body, 3, schedule=sched, operation=(jp.Concat(), jp.Add, jp.Max))

    ref_body = step(params, batch)
    got = jp.mpmd_jit_with_loop(step, cpu_mesh(2))(params, batch)
    assert_trees_equal(ref_body, got, exact=False, rtol=1e-6, atol=1e-7)


def test_schedule_stage_mismatch_is_reported():
    params, batch = mlp_params(4, 8), torch.randn(2, 2, 8)
    step = make_mlp_step(4, jp.Std1F1B(2), 2)  # 4 markers, schedule for 2 stages
    with pytest.raises(AssertionError, match="marks 4 stages but the schedule was built for 2"):
        jp.mpmd_jit_with_loop(step, cpu_mesh(2)).lower(params, batch)


def test_in_shardings_and_dump(tmp_path):
    sched = jp.Std1F1B(2)
    params, batch = mlp_params(2, 8), torch.randn(2, 2, 8)
    with config.dump_dir.set(str(tmp_path)):
        f = jp.mpmd_jit_with_loop(make_mlp_step(2, sched, 2), cpu_mesh(2), name="toy")
        compiled = f.lower(params, batch)
    (args, kwargs) = compiled.in_shardings
    assert args[0][0]["w1"].mesh_ids == frozenset({0}) and args[0][1]["w1"].mesh_ids == frozenset({1})
    assert args[1].mesh_ids == frozenset({0, 1})  # the batch feeds stage 0 and the loss on stage 1
    text = (tmp_path / "toy.global.0.program.txt").read_text()
    assert "task fwd_0__0" in text and "transfer#" in text
    assert "send#" in (tmp_path / "toy.local.0.rank0.program.txt").read_text()


@pytest.mark.parametrize("scarce", [False, True])
def test_licm_hoists_loop_invariant_casts(scarce):
    """With JAXPP_ENABLE_LICM a cast of the parameters written inside the loop body runs once before the loop
    (on each consumer rank) instead of once per microbatch; results are unchanged.  With scarce memory (the default)
    a *widening* cast that only the loop reads goes back inside: the small operand stays resident, not the large
    result (reference: src/jaxpp/licm.py:301-345)."""
    sched = jp.Std1F1B(2)
    params, batch = mlp_params(2, 8), torch.randn(4, 2, 8)

    def step(params, batch):
        def body(mb):
            def loss_fn(p):
                p = pytree.tree_map(lambda t: t.to(torch.float64), p)   # loop-invariant work
                return ((mlp_forward(p, mb.to(torch.float64), 2) - mb) ** 2).mean().float()

            return jp.value_and_grad(loss_fn)(params)

        return jp.treduce(body, batch, schedule=sched)

    ref = step(params, batch)
    plain = jp.mpmd_jit_with_loop(step, cpu_mesh(2)).lower(params, batch).program
    with config.enable_licm.set(True), config.licm_memory_scarce.set(scarce):
        f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
        hoisted = f.lower(params, batch).program
        got = f(params, batch)
    assert_trees_equal(ref, got, exact=True)

    def casts_in(prog, name):
        task = next(i for i in prog.instrs if isinstance(i, RunTask) and i.name == name)
        return task.code.src.count("T[%d]" % next(k for k, t in enumerate(task.code.targets) if "_to_copy" in str(t))) \
            if any("_to_copy" in str(t) for t in task.code.targets) else 0

    assert casts_in(plain, "fwd_0__0") >= 6
    if scarce:   # float32 -> float64 doubles the bytes: the casts stay with their consumers
        assert casts_in(hoisted, "fwd_0__0") >= 6
    else:
        assert casts_in(hoisted, "before_loop_r0") >= 5
        assert casts_in(hoisted, "fwd_0__0") == 1  # only the microbatch itself is still cast inside the loop


def test_licm_rules_narrowing_casts_fp8_and_cse():
    """Narrowing casts are hoisted even with scarce memory, casts to 8-bit floats never are, and identical pure ops
    are merged (reference: src/jaxpp/licm.py:66-126, 429-452)."""
    sched = jp.Std1F1B(2)
    params, batch = mlp_params(2, 8), torch.randn(4, 2, 8)

    def step(params, batch):
        def body(mb):
            def loss_fn(p):
                lo = pytree.tree_map(lambda t: t.to(torch.bfloat16).to(torch.float32), p)      # narrowing, then widening
                dup = pytree.tree_map(lambda t: t.to(torch.bfloat16).to(torch.float32), p)     # the same again
                q = pytree.tree_map(lambda t: t.to(torch.float8_e4m3fn).to(torch.float32), p)  # 8-bit round trip
                mixed = pytree.tree_map(lambda a, b, c: (a + b) * 0.5 + 0.0 * c, lo, dup, q)
                return ((mlp_forward(mixed, mb, 2) - mb) ** 2).mean()

            return jp.value_and_grad(loss_fn)(params)

        return jp.treduce(body, batch, schedule=sched)

    ref = step(params, batch)
    with config.enable_licm.set(True):
        f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
        prog = f.lower(params, batch).program
        got = f(params, batch)
    assert_trees_equal(ref, got, exact=True)
    src = {i.name: i.code for i in prog.instrs if isinstance(i, RunTask)}

    def count(code, dtype):
        return sum(1 for line in code.src.splitlines() if "dtype=" in line and f"C[{code.consts.index(dtype)}]" in line) \
            if dtype in code.consts else 0

    before, fwd = src["before_loop_r0"], src["fwd_0__0"]
    assert count(before, torch.bfloat16) >= 1 and count(fwd, torch.bfloat16) == 0       # hoisted once
    assert count(before, torch.float8_e4m3fn) == 0 and count(fwd, torch.float8_e4m3fn) >= 1   # stays in the loop
    plain = jp.mpmd_jit_with_loop(step, cpu_mesh(2)).lower(params, batch).program
    plain_fwd = next(i.code for i in plain.instrs if isinstance(i, RunTask) and i.name == "fwd_0__0")
    # without the pass every parameter is narrowed twice (lo and dup); with it once, before the loop
    assert count(plain_fwd, torch.bfloat16) == 2 * count(before, torch.bfloat16)


@pytest.mark.parametrize("schedule", [jp.Std1F1B(2), jp.Interleaved1F1B(4, 2), jp.ZeroBubble(2)], ids=["1f1b", "interleaved", "zb"])
def test_dropout_inside_the_pipelined_loop_draws_the_same_numbers(schedule):
    """Random numbers inside the microbatch loop (the reference's tests/functional_testing/test_dropout_enabled.py):
    the mask is a function of (seed, microbatch, layer), so the scheduled program -- stages on different ranks,
    backward tasks regenerating their masks, ZeroBubble's split backward -- must reproduce the sequential step
    bit for bit, and a different seed must change the result."""
    n_stages, n_mb = schedule.num_stages, 4
    params = mlp_params(n_stages, 8)
    batch = torch.randn(n_mb, 3, 8, generator=torch.Generator().manual_seed(3))

    def make_step(seed):
        def step(params, batch, base_seed):
            def body(i):
                mb = jp.take(batch, i)
                seed_i = base_seed + i                       # a fresh stream per microbatch

                def loss_fn(p):
                    x = mb
                    for layer, q in enumerate(p):
                        h = ops.gelu(ops.linear(x, q["w1"], q["b1"]))
                        h = ops.dropout(h, 0.25, seed_i, layer)
                        x = ops.layernorm(x + ops.linear(h, q["w2"], None), q["g"], q["b"], 1e-5)[0]
                        x = jp.mark_stage_end(x)
                    return ((x - mb) ** 2).mean()

                return jp.value_and_grad(loss_fn)(params)

            return jp.treduce_i(body, n_mb, schedule=schedule)

        return step

    seed = torch.tensor(1234, dtype=torch.int64)
    step = make_step(seed)
    ref = step(params, batch, seed)
    got = jp.mpmd_jit_with_loop(step, cpu_mesh(2))(params, batch, seed)
    assert_trees_equal(ref, got, exact=True)
    other = step(params, batch, seed + 1)
    assert not torch.equal(leaves(other)[0], leaves(ref)[0])


def test_weight_gradients_sink_into_the_loop_accumulators():
    """Weight gradients that only feed the loop's Add accumulation are added into the accumulator by the producing
    op; the scheduled program marks those outputs, the accumulation step becomes a no-op for them, and the result
    is identical to the literal produce-then-add form."""
    sched = jp.Std1F1B(2)
    params = mlp_params(2, 8)
    batch = torch.randn(4, 3, 8, generator=torch.Generator().manual_seed(7))
    step = make_mlp_step(2, sched, 4)
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
    compiled = f.lower(params, batch)
    tasks = [i for i in compiled.program.instrs if isinstance(i, RunTask)]
    sunk = [i for i in tasks if i.sinks]
    assert sunk, "no task output was recognised as a weight-gradient sink"
    assert all(t.task_type is None or "bwd" in str(t.task_type).lower() or "BWD" in str(t.task_type) for t in sunk)
    n_w = sum(1 for p in params for k in p if k in ("w1", "w2"))
    assert max(len(t.sinks) for t in sunk) <= n_w
    got = f(params, batch)
    with config.wgrad_sinks.set(False):
        g = jp.mpmd_jit_with_loop(make_mlp_step(2, sched, 4), cpu_mesh(2))
        plain = g.lower(params, batch)
        assert not any(i.sinks for i in plain.program.instrs if isinstance(i, RunTask))
        ref = g(params, batch)
    eager = step(params, batch)
    assert_trees_equal(eager, got, exact=True)
    assert_trees_equal(eager, ref, exact=True)


def test_norm_backward_absorbs_the_residual_gradient_add():
    """Pre-norm residual blocks: ``norm_bwd`` + ``add`` is rewritten into one op; the program still matches the eager
    step bit for bit (the fused op rounds like the two separate kernels)."""
    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf

    cfg = tf.ModelConfig("llama", vocab=128, d_model=32, n_layers=2, n_heads=2, n_kv_heads=2, ffn=64, seq=16, n_stages=2,
                         tp=1, dtype=torch.float32)
    sched = jp.Std1F1B(2)
    state = lt.init_state(cfg, sched, "cpu")
    g = torch.Generator().manual_seed(0)
    tok, lab = torch.randint(0, 128, (2, 2, 16), generator=g), torch.randint(0, 128, (2, 2, 16), generator=g)
    step = lt.make_train_step(cfg, sched, lt.Hyper(inplace_update=False))
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
    compiled = f.lower(state, tok, lab)
    used = set()
    for ins in compiled.program.instrs:
        if isinstance(ins, RunTask):
            used |= {str(t) for t in ins.code.targets}
    assert "b200.rmsnorm_bwd_add.default" in used
    assert_trees_equal(step(state, tok, lab), f(state, tok, lab), exact=True)
    with config.fuse_norm_backward_adds.set(False):
        plain = jp.mpmd_jit_with_loop(lt.make_train_step(cfg, sched, lt.Hyper(inplace_update=False)), cpu_mesh(2))
        used2 = set()
        for ins in plain.lower(state, tok, lab).program.instrs:
            if isinstance(ins, RunTask):
                used2 |= {str(t) for t in ins.code.targets}
        assert "b200.rmsnorm_bwd_add.default" not in used2


def test_loop_body_constant_needs_the_relaxed_clustering_flag():
    """A value made inside the loop body that neither depends on nor feeds a stage (a literal returned next to the
    loss) is refused under conservative clustering and joins the last cluster with the flag off; custom reduction
    ops per output (the case of the reference's tests/test_transformations.py:218-251)."""
    g = torch.Generator().manual_seed(7)
    sched = jp.Std1F1B(1)
    w, X, Y = torch.rand(10, 10, generator=g), torch.rand(2, 10, generator=g), torch.rand(2, 10, generator=g)

    def step(w, X, Y):
        def body(d):
            x, y = d
            loss, grad = jp.value_and_grad(lambda w: ((jp.mark_stage_end(w @ x) - y) ** 2).mean())(w)
            return loss, grad, torch.tensor(1.0)

        return jp.treduce(body, (X, Y), schedule=sched, operation=(jp.Concat(), jp.Add, jp.Add))

    ref = step(w, X, Y)
    with pytest.raises(AssertionError, match="neither depends on nor feeds"):
        jp.mpmd_jit_with_loop(step, cpu_mesh(1))(w, X, Y)
    with config.conservative_loop_clustering.set(False):
        got = jp.mpmd_jit_with_loop(step, cpu_mesh(1))(w, X, Y)
    assert_trees_equal(ref, got, exact=True)
    assert float(local(got[2])) == 2.0


def test_parallel_branches_each_end_a_stage():
    """Two stages that both read the microbatch and do not depend on each other, merged by a third; the step also
    returns a Python constant and passes an input through (the case of the reference's
    tests/test_transformations.py:254-322)."""
    g = torch.Generator().manual_seed(7)
    sched = jp.Eager1F1B(3)
    ws = tuple(torch.rand(10, 10, generator=g) for _ in range(3))
    X, Y = torch.rand(5, 10, generator=g), torch.rand(5, 10, generator=g)

    def predict(params, x):
        w1, w2, w3 = params
        a = jp.mark_stage_end(w1 @ x)
        b = jp.mark_stage_end(w2 @ x)
        return jp.mark_stage_end(w3 @ (a + b))

    def step(params, X, Y):
        def body(d):
            x, y = d
            return jp.value_and_grad(lambda p: ((predict(p, x) - y) ** 2).mean())(params)

        losses, grads = jp.treduce(body, (X, Y), schedule=sched)
        return (losses, pytree.tree_map(lambda p, gg: p - 0.1 * gg, params, grads)), 5, X

    ref = step(ws, X, Y)
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(3))
    got = f(ws, X, Y)
    assert got[1] == 5
    assert_trees_equal((ref[0], ref[2]), (got[0], got[2]), exact=False, rtol=1e-5, atol=1e-6)
    verify_program(f.lower(ws, X, Y).program)


def _marked_mlp(params, x):
    first_stage_output = None
    for i, (w, b) in enumerate(params):
        if i == 1:
            first_stage_output = x
        x = jp.mark_stage_end(torch.tanh(x @ w + b))
    return x, first_stage_output


def _late_param(p, X):
    return _marked_mlp(p, X)[0] + p[1][1]


def _early_value(p, X):
    return _marked_mlp(p, X)[1] + p[1][1]


def _select(p, X):
    preds, early = _marked_mlp(p, X)
    picked = torch.where((preds < 0).any(), early, early * 2 + torch.zeros_like(early))
    return picked + p[0][1]


@pytest.mark.parametrize("fn,rank", [(_late_param, 3), (_early_value, 0), (_select, 3)])
def test_forward_only_pipeline_with_values_used_across_stages(fn, rank):
    """Forward-only pipelines whose result uses a parameter of an earlier stage after the last marker, returns a
    value of the first stage, or selects between stages' values (the cases of the reference's
    tests/test_transformations.py:331-435); the result lives on the rank that computes it."""
    g = torch.Generator().manual_seed(3)
    params = [(torch.rand(10, 10, generator=g), torch.rand(10, generator=g)) for _ in range(4)]
    X = torch.rand(6, 10, generator=g)
    got = jp.mpmd_jit_by_yield(fn, cpu_mesh(4))(params, X)
    torch.testing.assert_close(local(got), fn(params, X), rtol=1e-6, atol=1e-6)
    assert got.mpmd_idxs == (rank,)


def test_loop_without_after_loop_computation():
    """The step returns the reduced values as they are: nothing runs after the loop."""
    sched = jp.Eager1F1B(3)
    params, batch = mlp_params(3, 8), torch.randn(5, 2, 8, generator=torch.Generator().manual_seed(2))

    def step(params, batch):
        def body(mb):
            return jp.value_and_grad(lambda p: ((mlp_forward(p, mb, 3) - mb) ** 2).mean())(params)

        return jp.treduce(body, batch, schedule=sched)

    assert_trees_equal(step(params, batch), jp.mpmd_jit_with_loop(step, cpu_mesh(3))(params, batch), exact=True)


@pytest.mark.parametrize("pp", [1, 2])
def test_microbatch_inputs_passed_through_the_loop(pp):
    """The body returns its own inputs next to the loss (stacked over microbatches again by ``Concat``), one of them
    also used after the last marker (the case of the reference's tests/functional_testing/test_passthrough_vars.py:
    36-75)."""
    g = torch.Generator().manual_seed(1)
    ws = [torch.randn(100, 100, generator=g) * 0.1 for _ in range(4)]
    X, Yin = torch.randn(3, 10, 100, generator=g), torch.randn(3, 10, 100, generator=g)
    T = torch.randint(0, 100, (3, 10), generator=g)
    sched = jp.Std1F1B(pp)

    def step(ws, X, Yin, T):
        def body(d):
            (x, y), t = d

            def loss_fn(ws):
                out = x
                for i, w in enumerate(ws):
                    out = out @ w
                    if pp == 2 and i == 1:
                        out = jp.mark_stage_end(out)
                out = jp.mark_stage_end(out)
                logits = out + y
                return ops.cross_entropy(logits, t)[0].mean(), (logits, x, y)

            return jp.value_and_grad(loss_fn, has_aux=True)(ws)

        (loss, (logits, x, y)), grads = jp.treduce(body, ((X, Yin), T), schedule=sched)
        return [w - 0.1 * gg for w, gg in zip(ws, grads)], loss.mean(), x, y, logits

    ref = step(ws, X, Yin, T)
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(pp))
    got = f(ws, X, Yin, T)
    assert_trees_equal(ref, got, exact=True)
    assert torch.equal(local(got[2]), X) and torch.equal(local(got[3]), Yin)
    verify_program(f.lower(ws, X, Yin, T).program)


# ---- donation, static arguments, per-rank programs in one process -----------------------------------------------------
def test_donated_arguments_are_freed_at_their_last_use():
    """``donate_argnums``: program inputs the caller gave up are deleted (or handed to their last task) after their last
    use on every rank instead of living for the whole step; arrays passed for them read as deleted afterwards
    (reference: infer_donation, src/jaxpp/core.py:1732-1809; jit arguments :3892-3923)."""
    from jaxpp_b200.compiler.program import Delete

    sched = jp.Std1F1B(2)
    params, batch = mlp_params(2, 8), torch.randn(4, 2, 8)
    step = make_mlp_step(2, sched, 4)
    ref = step(params, batch)
    kept = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
    gave = jp.mpmd_jit_with_loop(step, cpu_mesh(2), donate_argnums=(0,))
    p_kept, p_gave = kept.lower(params, batch).program, gave.lower(params, batch).program
    param_vids = {vid for k, (vid, _) in enumerate(p_gave.inputs) if k < len(leaves(params))}

    def freed(prog):
        out = set()
        for i in prog.instrs:
            if isinstance(i, Delete):
                out.update(v for v in i.vids if v in param_vids)
            if isinstance(i, RunTask):
                out.update(v for v, d in zip(i.ins, i.donate) if d and v in param_vids)
        return out

    assert not freed(p_kept) and freed(p_gave) == param_vids
    verify_program(p_gave)
    first = gave(params, batch)                       # plain tensors: the caller still owns them
    assert_trees_equal(ref, first, exact=True)
    state = first[1]                                  # MpmdArrays: donated on the next call
    ref2 = step(pytree.tree_map(local, state), batch)
    second = gave(state, batch)
    assert_trees_equal(ref2, second, exact=True)
    assert all(a.is_deleted() for a in leaves(state))
    with pytest.raises(ValueError):
        jp.mpmd_jit_with_loop(step, cpu_mesh(2), donate_argnums=(5,)).lower(params, batch)


def test_donation_lowers_peak_memory_of_a_step():
    """Live bytes over the instruction list: with the old state donated, old and new parameters never coexist in full."""
    import math

    from jaxpp_b200.compiler.program import Delete

    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf

    sched = jp.Std1F1B(2)
    cfg = tf.ModelConfig("llama", vocab=64, d_model=64, n_layers=2, n_heads=2, n_kv_heads=2, ffn=128, seq=8, n_stages=2,
                         dtype=torch.float32)
    step = lt.make_train_step(cfg, sched, lt.Hyper(inplace_update=False))     # the new state is fresh memory
    state = lt.init_state(cfg, sched, "cpu")
    tokens = torch.randint(0, 64, (2, 1, 8))

    def peak_bytes(prog):
        size = lambda v: math.prod(prog.values[v].shape) * prog.values[v].dtype.itemsize
        live = [set(v for v, ranks in prog.inputs if r in ranks) for r in range(prog.n_ranks)]
        peak = [sum(size(v) for v in s) for s in live]
        for i in prog.instrs:
            r = i.rank
            if isinstance(i, RunTask):
                live[r] -= {v for v, d in zip(i.ins, i.donate) if d}
                live[r] |= {v for v in i.outs if v >= 0}
            elif isinstance(i, Delete):
                live[r] -= set(i.vids)
            elif isinstance(i, Transfer):
                live[i.dst] |= set(i.vids)
            elif hasattr(i, "out") and isinstance(getattr(i, "out"), int):
                live[r].add(i.out)
            peak[r] = max(peak[r], sum(size(v) for v in live[r]))
        return max(peak)

    kept = jp.mpmd_jit_with_loop(step, cpu_mesh(2)).lower(state, tokens, tokens).program
    gave = jp.mpmd_jit_with_loop(step, cpu_mesh(2), donate_argnums=(0,)).lower(state, tokens, tokens).program
    # kept: old and new (parameters, master weights, two moments) coexist after the optimizer task; donated: one set
    assert peak_bytes(gave) < 0.75 * peak_bytes(kept)


def test_static_arguments_are_constants_and_must_not_hold_arrays():
    sched = jp.Std1F1B(2)
    params, batch = mlp_params(2, 8), torch.randn(4, 2, 8)

    def step(params, batch, scale):
        loss, new = make_mlp_step(2, sched, 4)(params, batch)
        return loss * scale, new

    f = jp.mpmd_jit_with_loop(step, cpu_mesh(2), static_argnums=(2,))
    assert_trees_equal(step(params, batch, 2.0), f(params, batch, 2.0), exact=True)
    assert_trees_equal(step(params, batch, 3.0), f(params, batch, 3.0), exact=True)   # a new constant: a new program
    assert len(f._cache) == 2
    with pytest.raises(TypeError):
        jp.mpmd_jit_with_loop(step, cpu_mesh(2), static_argnums=(1,)).lower(params, batch, 2.0)


@pytest.mark.parametrize("pp,schedule,n_mb", [(2, jp.Std1F1B(2), 4), (2, jp.Interleaved1F1B(4, 2), 4), (4, jp.ZeroBubble(4), 6),
                                              (2, jp.DualPipeV(4, 2), 4)], ids=["1f1b", "interleaved", "zb", "dualpipev"])
def test_force_mpmdify_runs_the_per_rank_programs_in_one_process(pp, schedule, n_mb):
    """``JAXPP_DEBUG_FORCE_MPMDIFY``: the per-rank instruction lists of the multi-process path (send / recv /
    send_done / all_reduce per rank), run as threads of one process, give the results of the global program."""
    params = mlp_params(schedule.num_stages, 16)
    batch = torch.randn(n_mb, 4, 16, generator=torch.Generator().manual_seed(1))
    step = make_mlp_step(schedule.num_stages, schedule, n_mb)
    ref = step(params, batch)
    with config.debug_force_mpmdify.set(True):
        f = jp.mpmd_jit_with_loop(step, cpu_mesh(pp))
        got = f(params, batch)
        again = f(got[1], batch)
    assert_trees_equal(ref, got, exact=True)
    assert_trees_equal(step(pytree.tree_map(local, got[1]), batch), again, exact=True)


def test_force_mpmdify_with_cross_rank_collectives_and_a_failing_rank():
    sched = jp.Std1F1B(2)
    g = torch.Generator().manual_seed(3)
    params = {"emb": torch.randn(8, 8, generator=g) * 0.3, "mid": torch.randn(8, 8, generator=g) * 0.3}
    batch = torch.randn(4, 4, 8, generator=g)

    def step(params, batch):
        def body(mb):
            def loss_fn(p):
                x = jp.mark_stage_end(ops.gelu(ops.linear(mb, p["emb"], None)))
                x = ops.linear(ops.linear(x, p["mid"], None), p["emb"], None)   # tied weight: cross-rank all-reduce
                return (jp.mark_stage_end(x) ** 2).mean() / 4

            return jp.value_and_grad(loss_fn)(params)

        loss, grads = jp.treduce(body, batch, schedule=sched)
        norms = jp.cross_mpmd_stack([grads["emb"].pow(2).sum().reshape(1), grads["mid"].pow(2).sum().reshape(1)], axis=0)
        return loss, pytree.tree_map(lambda p, gr: p - 0.5 * gr, params, grads), norms

    ref = step(params, batch)
    global_run = jp.mpmd_jit_with_loop(step, cpu_mesh(2))(params, batch)
    with config.debug_force_mpmdify.set(True):
        f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
        got = f(params, batch)
        assert_trees_equal(ref, got, exact=False)           # the tied gradient is summed in a different order
        assert_trees_equal(pytree.tree_map(local, global_run), got, exact=True)   # same as the global program, bit for bit
        from jaxpp_b200 import fault

        fault.set_fault_plan(fault.FaultPlan(raise_in_task="bwd_1__2", on_rank=1))
        try:
            with pytest.raises(fault.InjectedFault):   # the failing rank's error, not the others' "partner failed"
                f(params, batch)
        finally:
            fault.set_fault_plan(None)
