"""Model families through the whole stack on CPU: pipelined step == un-pipelined step."""
import pytest
import torch
from torch.utils import _pytree as pytree

import jaxpp_b200 as jp
from jaxpp_b200.models import lm_trainer as lt
from jaxpp_b200.models import transformer as tf

from helpers import assert_trees_equal, local


def cpu_mesh(pp):
    return jp.MpmdMesh.create({"mpmd": pp, "data": 1, "model": 1}, kind="cpu", multi_process=False)


def test_encoder_example_matches_unpipelined():
    """The CPU plumbing configuration: 4-layer post-LN encoder (hidden 256, 4 heads, FFN 1024, GELU), fp32,
    2 stages on 2 ranks, Std1F1B, 4 microbatches of 8 x 128, MSE against the input, Adam."""
    cfg = tf.bert_example(n_stages=2)
    sched = jp.Std1F1B(2)
    n_mb = 4
    params = tf.init_params(cfg, "cpu", seed=1)
    hidden = torch.randn(n_mb * 8, 128, 256, generator=torch.Generator().manual_seed(0)).view(n_mb, 8, 128, 256)
    m = pytree.tree_map(torch.zeros_like, params)
    v = pytree.tree_map(torch.zeros_like, params)
    from jaxpp_b200.ops import core as ops

    def step(params, m, v, count, batch):
        def body(mb):
            def loss_fn(p):
                out = tf.encoder_forward(cfg, p, mb)
                return ((out - mb) ** 2).mean() / n_mb

            return jp.value_and_grad(loss_fn)(params)

        losses, grads = jp.treduce(body, batch, schedule=sched)
        new_count = count + 1
        upd = pytree.tree_map(
            lambda p, g, mm, vv: ops.adamw(p, g, mm, vv, new_count, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1.0, torch.float32)[:3],
            params, grads, m, v)
        pick = lambda k: pytree.tree_map(lambda p, u: u[k], params, upd, is_leaf=lambda x: isinstance(x, tuple))
        return losses, grads, pick(0), pick(1), pick(2), new_count

    count = torch.zeros((), dtype=torch.int64)
    ref = step(params, m, v, count, hidden)
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
    got = f(params, m, v, count, hidden)
    assert_trees_equal(ref, got, exact=True)
    assert got[0].mpmd_idxs == (1,) and int(got[5]) == 1 and got[5].mpmd_idxs == (0, 1)
    # a second step from the returned state (MpmdArrays go straight back in)
    ref2 = step(ref[2], ref[3], ref[4], ref[5], hidden)
    got2 = f(got[2], got[3], got[4], got[5], hidden)
    assert_trees_equal(ref2, got2, exact=True)
    assert torch.isfinite(local(got2[0])).all()


@pytest.mark.parametrize("family,schedule,pp", [
    ("llama", jp.Interleaved1F1B(4, 2), 2),
    ("gpt2", jp.Std1F1B(2), 2),
    ("llama", jp.ZeroBubble(2), 2),
])
def test_lm_trainer_matches_unpipelined(family, schedule, pp):
    cfg = tf.ModelConfig(family, vocab=250, d_model=64, n_layers=4, n_heads=4, n_kv_heads=2 if family == "llama" else 4,
                         ffn=128, seq=32, n_stages=schedule.num_stages, dtype=torch.float32)
    hyper = lt.Hyper(lr=1e-2, inplace_update=False)
    step = lt.make_train_step(cfg, schedule, hyper)
    state = lt.init_state(cfg, schedule, "cpu")
    g = torch.Generator().manual_seed(5)
    n_mb = 4
    tokens = torch.randint(0, cfg.vocab, (n_mb, 2, cfg.seq), generator=g)
    labels = torch.randint(0, cfg.vocab, (n_mb, 2, cfg.seq), generator=g)
    ref_state, ref_losses = step(state, tokens, labels)
    f = jp.mpmd_jit_with_loop(step, cpu_mesh(pp))
    got_state, got_losses = f(state, tokens, labels)
    assert_trees_equal((ref_state, ref_losses), (got_state, got_losses), exact=True)
    owners = lt.owner_ranks(cfg, schedule)
    assert got_state["params"]["embed"].mpmd_idxs == (owners["embed"],)
    assert got_state["params"]["layers"]["003"]["wqkv"].mpmd_idxs == (owners[3],)
    assert abs(float(local(got_losses).mean()) - torch.log(torch.tensor(float(cfg.padded_vocab)))) < 0.5


def test_tied_embeddings_across_stages():
    sched = jp.Std1F1B(2)
    cfg = tf.ModelConfig("llama", vocab=128, d_model=32, n_layers=2, n_heads=2, n_kv_heads=2, ffn=64, seq=16, n_stages=2,
                         dtype=torch.float32, tie_embeddings=True)
    step = lt.make_train_step(cfg, sched, lt.Hyper(lr=1e-2, inplace_update=False))
    state = lt.init_state(cfg, sched, "cpu")
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, 128, (2, 2, 16), generator=g)
    labels = torch.randint(0, 128, (2, 2, 16), generator=g)
    ref = step(state, tokens, labels)
    got = jp.mpmd_jit_with_loop(step, cpu_mesh(2))(state, tokens, labels)
    assert got[0]["params"]["embed"].mpmd_idxs == (0, 1)  # the tied table lives on both ranks
    assert_trees_equal(ref, got, exact=False, rtol=1e-5, atol=1e-6)


def test_mixtral_moe_pipelined_matches_unpipelined():
    sched = jp.DualPipeV(4, 2)
    cfg = tf.ModelConfig("mixtral", vocab=128, d_model=32, n_layers=4, n_heads=2, n_kv_heads=1, ffn=64, seq=16, n_stages=4,
                         dtype=torch.float32, n_experts=4, top_k=2, capacity_factor=2.0)
    step = lt.make_train_step(cfg, sched, lt.Hyper(lr=1e-2, inplace_update=False))
    state = lt.init_state(cfg, sched, "cpu")
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, 128, (4, 2, 16), generator=g)
    labels = torch.randint(0, 128, (4, 2, 16), generator=g)
    ref = step(state, tokens, labels)
    got = jp.mpmd_jit_with_loop(step, cpu_mesh(2))(state, tokens, labels)
    assert_trees_equal(ref, got, exact=True)
    assert got[0]["params"]["layers"]["003"]["e_up"].mpmd_idxs == (0,)  # V placement: stage 3 is back on rank 0
    # the router gets a gradient from both the task loss and the load-balancing term
    assert not torch.equal(local(got[0]["params"]["layers"]["000"]["router"]), state["params"]["layers"]["000"]["router"])


def test_activation_recompute_matches_and_moves_forward_ops_into_backward():
    from jaxpp_b200.compiler.program import RunTask

    sched = jp.ZeroBubble(2)
    kw = dict(vocab=128, d_model=32, n_layers=2, n_heads=2, n_kv_heads=2, ffn=64, seq=16, n_stages=2, dtype=torch.float32)
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, 128, (2, 2, 16), generator=g)
    labels = torch.randint(0, 128, (2, 2, 16), generator=g)
    outs, progs = [], []
    for rec in (False, True):
        cfg = tf.ModelConfig("llama", recompute=rec, **kw)
        step = lt.make_train_step(cfg, sched, lt.Hyper(lr=1e-2, inplace_update=False))
        state = lt.init_state(cfg, sched, "cpu")
        f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
        outs.append(f(state, tokens, labels))
        progs.append(f.lower(state, tokens, labels).program)
    assert_trees_equal(pytree.tree_map(local, outs[0], is_leaf=lambda x: isinstance(x, jp.MpmdArray)), outs[1], exact=True)

    def n_attn(prog, name):
        t = next(i for i in prog.instrs if isinstance(i, RunTask) and i.name == name)
        return sum("b200.attention.default" in str(x) for x in t.code.targets)

    assert n_attn(progs[0], "bwdA_1__0") == 0 and n_attn(progs[1], "bwdA_1__0") == 1  # forward re-run inside backward
    # and the forward task hands fewer activations to the backward task
    fwd = lambda prog: next(i for i in prog.instrs if isinstance(i, RunTask) and i.name == "fwd_1__0")
    assert len(fwd(progs[1]).outs) < len(fwd(progs[0]).outs)
    # the FIRST stage too: no backward marker follows its backward pass, and its re-run forward reads forward values
    # only -- it must still run in the backward task, not a second time in the forward task
    first_bwd = next(i.name for i in progs[0].instrs if isinstance(i, RunTask) and i.name.startswith("bwd") and "_0__0" in i.name)
    assert n_attn(progs[0], "fwd_0__0") == n_attn(progs[1], "fwd_0__0") == 1
    assert n_attn(progs[0], first_bwd) == 0 and n_attn(progs[1], first_bwd) == 1
    fwd0 = lambda prog: next(i for i in prog.instrs if isinstance(i, RunTask) and i.name == "fwd_0__0")
    assert len(fwd0(progs[1]).outs) < len(fwd0(progs[0]).outs)


def test_cse_does_not_undo_activation_recompute_unless_asked():
    """With common-subexpression elimination on, the re-run forward of a recomputed block equals the forward pass op for
    op; merging them would hand every activation from the forward task to the backward task again."""
    from jaxpp_b200.compiler.program import RunTask
    from jaxpp_b200.utils import config

    sched = jp.Std1F1B(2)
    kw = dict(vocab=128, d_model=32, n_layers=2, n_heads=2, n_kv_heads=2, ffn=64, seq=16, n_stages=2, dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, 128, (2, 2, 16), generator=g)
    labels = torch.randint(0, 128, (2, 2, 16), generator=g)
    cfg = tf.ModelConfig("llama", recompute=True, **kw)

    def n_fwd_outs(**flags):
        step = lt.make_train_step(cfg, sched, lt.Hyper(lr=1e-2, inplace_update=False))
        state = lt.init_state(cfg, sched, "cpu")
        with config.enable_licm.set(flags.get("licm", False)), config.disable_prevent_cse.set(flags.get("lift", False)):
            f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
            prog = f.lower(state, tokens, labels).program
            out = f(state, tokens, labels)
        fwd0 = next(i for i in prog.instrs if isinstance(i, RunTask) and i.name == "fwd_0__0")
        return len(fwd0.outs), out

    plain, ref = n_fwd_outs()
    kept, got = n_fwd_outs(licm=True)
    lifted, got2 = n_fwd_outs(licm=True, lift=True)
    assert kept <= plain < lifted
    assert_trees_equal(pytree.tree_map(local, ref, is_leaf=lambda x: isinstance(x, jp.MpmdArray)), got, exact=True)
    assert_trees_equal(pytree.tree_map(local, ref, is_leaf=lambda x: isinstance(x, jp.MpmdArray)), got2, exact=True)


@pytest.mark.parametrize("family,schedule,tied", [
    ("llama", jp.Interleaved1F1B(4, 2), False), ("gpt2", jp.Std1F1B(2), True), ("llama", jp.ZeroBubble(2), False),
])
def test_gradient_clipping_by_global_norm(family, schedule, tied):
    """``Hyper.clip_grad_norm``: per-rank sums of squares meet in a cross-stage all-reduce; the first Adam moment after
    one step is (1 - beta1) * clipped gradient, so its norm shows the threshold."""
    cfg = tf.ModelConfig(family, vocab=250, d_model=64, n_layers=4, n_heads=4, n_kv_heads=2 if family == "llama" else 4,
                         ffn=128, seq=32, n_stages=schedule.num_stages, dtype=torch.float32, tie_embeddings=tied)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab, (4, 2, cfg.seq), generator=g)
    labels = torch.randint(0, cfg.vocab, (4, 2, cfg.seq), generator=g)
    norms = {}
    for clip in (None, 0.05):
        step = lt.make_train_step(cfg, schedule, lt.Hyper(lr=1e-2, inplace_update=False, clip_grad_norm=clip))
        state = lt.init_state(cfg, schedule, "cpu")
        ref_state, _ = step(state, tokens, labels)
        got_state, _ = jp.mpmd_jit_with_loop(step, cpu_mesh(2))(state, tokens, labels)
        assert_trees_equal(ref_state, got_state, exact=not tied, rtol=1e-5, atol=1e-6)
        norms[clip] = float(torch.cat([t.reshape(-1) for t in pytree.tree_leaves(ref_state["m"])]).norm() / (1 - 0.9))
    assert norms[None] > 0.5 and abs(norms[0.05] - 0.05) < 1e-4


def test_activation_recompute_of_mixture_of_experts_blocks():
    """A block with two outputs (hidden state and load-balancing loss) under recompute: same results as without, the
    forward task keeps fewer activations (what lets the Mixtral benchmark configuration fit in 180 GB)."""
    from jaxpp_b200.compiler.program import RunTask

    sched = jp.DualPipeV(4, 2)
    kw = dict(vocab=128, d_model=32, n_layers=4, n_heads=2, n_kv_heads=2, ffn=64, seq=16, n_stages=4, dtype=torch.float32,
              n_experts=4, top_k=2, capacity_factor=4.0, aux_coef=0.01)
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, 128, (4, 2, 16), generator=g)
    labels = torch.randint(0, 128, (4, 2, 16), generator=g)
    outs, progs = [], []
    for rec in (False, True):
        cfg = tf.ModelConfig("mixtral", recompute=rec, **kw)
        step = lt.make_train_step(cfg, sched, lt.Hyper(lr=1e-2, inplace_update=False))
        state = lt.init_state(cfg, sched, "cpu")
        f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
        outs.append(f(state, tokens, labels))
        progs.append(f.lower(state, tokens, labels).program)
    assert_trees_equal(pytree.tree_map(local, outs[0], is_leaf=lambda x: isinstance(x, jp.MpmdArray)), outs[1],
                       exact=False, rtol=1e-5, atol=1e-6)
    fwd = lambda prog: next(i for i in prog.instrs if isinstance(i, RunTask) and i.name.startswith("fwd_1"))
    assert len(fwd(progs[1]).outs) < len(fwd(progs[0]).outs)


@pytest.mark.parametrize("family,schedule,pp,stage_layers,recompute", [
    ("llama", jp.Interleaved1F1B(4, 2), 2, (1.5, 1, 1, 0.5), False),   # boundaries inside blocks 1 and 3
    ("gpt2", jp.Std1F1B(2), 2, (3, 1), False),                        # whole blocks, unequal
    ("llama", jp.ZeroBubble(2), 2, (2.5, 1.5), True),                 # cut block recomputed as two halves
    ("mixtral", jp.DualPipeV(4, 2), 2, (1, 1.5, 0.5, 1), False),
])
def test_unequal_and_half_block_stages_match_unpipelined(family, schedule, pp, stage_layers, recompute):
    extra = dict(n_experts=4, top_k=2, capacity_factor=2.0) if family == "mixtral" else {}
    cfg = tf.ModelConfig(family, vocab=250, d_model=64, n_layers=4, n_heads=4, n_kv_heads=2 if family != "gpt2" else 4,
                         ffn=128, seq=32, n_stages=schedule.num_stages, dtype=torch.float32, stage_layers=stage_layers,
                         recompute=recompute, **extra)
    step = lt.make_train_step(cfg, schedule, lt.Hyper(lr=1e-2, inplace_update=False))
    state = lt.init_state(cfg, schedule, "cpu")
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab, (4, 2, cfg.seq), generator=g)
    labels = torch.randint(0, cfg.vocab, (4, 2, cfg.seq), generator=g)
    ref = step(state, tokens, labels)
    got = jp.mpmd_jit_with_loop(step, cpu_mesh(pp))(state, tokens, labels)
    assert_trees_equal(ref, got, exact=True)
    owners = lt.owner_ranks(cfg, schedule)
    for name, layer in got[0]["params"]["layers"].items():
        for key, leaf in layer.items():
            assert leaf.mpmd_idxs == (lt.owner_of(owners, int(name), key),), (name, key)


def test_stage_layers_validation_and_balancing():
    with pytest.raises(ValueError):
        tf.llama2_7b(n_stages=8, stage_layers=(4,) * 7 + (5,))
    with pytest.raises(ValueError):
        tf.llama2_7b(n_stages=8, stage_layers=(4.25, 3.75) + (4,) * 6)
    cfg = tf.llama2_7b(n_stages=8, stage_layers=(4, 4, 4, 4, 4, 4, 4.5, 3.5))
    assert cfg.stage_ends_half == (8, 16, 24, 32, 40, 48, 57, 64)
    assert cfg.stage_of_param(28, "wqkv") == 6 and cfg.stage_of_param(28, "w_up") == 7
    sched = jp.Interleaved1F1B(8, 4)
    sizes = tf.balanced_stage_layers(32, 8, sched.get_mpmd_idx, 4, last_extra=0.73)
    equal = tf.rank_loads((4,) * 8, sched.get_mpmd_idx, 4, 0.36, 0.0, 0.73)
    best = tf.rank_loads(sizes, sched.get_mpmd_idx, 4, 0.36, 0.0, 0.73)
    assert abs(sum(sizes) - 32) < 1e-9 and max(best) < max(equal) - 0.3
    # per-process state with a cut block: each pipeline rank holds only the half it runs
    small = tf.ModelConfig("llama", vocab=64, d_model=32, n_layers=2, n_heads=2, n_kv_heads=2, ffn=64, seq=8, n_stages=2,
                           dtype=torch.float32, stage_layers=(1.5, 0.5))
    s0 = lt.init_state(small, jp.Std1F1B(2), "cpu", my_rank=0)
    s1 = lt.init_state(small, jp.Std1F1B(2), "cpu", my_rank=1)
    assert isinstance(s0["params"]["layers"]["001"]["wqkv"], torch.Tensor)
    assert isinstance(s0["params"]["layers"]["001"]["w_up"], jp.ShapeDtypeStruct)
    assert isinstance(s1["params"]["layers"]["001"]["w_up"], torch.Tensor)
    assert isinstance(s1["params"]["layers"]["001"]["wqkv"], jp.ShapeDtypeStruct)


def test_launch_bound_configurations_are_told_apart():
    """One GPT-2-XL sequence per replica makes kernels shorter than the Python that launches them (stages then cost
    their number of kernels: equal stages); the large shapes are bound by the GPU (stages cost their FLOPs)."""
    from jaxpp_b200 import configs

    seen = {}
    for name, per_rank in (("gpt2xl_pp2dp4", 1), ("llama7b_pp4tp2", 4), ("mixtral8x7b_pp2ep4", 2), ("llama70b_pp4tp2", 1)):
        cfg = configs.get(name).model_config()
        seen[name] = tf.launch_bound(cfg, per_rank * cfg.seq)
    assert seen == {"gpt2xl_pp2dp4": True, "llama7b_pp4tp2": False, "mixtral8x7b_pp2ep4": False, "llama70b_pp4tp2": False}
    attn_share, head_extra, first_extra = tf.stage_cost_model(configs.get("llama7b_pp4tp2").model_config())
    assert 0.3 < attn_share < 0.6 and 0.4 < head_extra < 0.8 and first_extra == 0.0


def test_zero_bubble_split_bounds_what_stays_alive_until_the_weight_gradient_half():
    """ZeroBubble with full recompute: the recomputed inputs and the activation gradients of every linear live from the
    activation-gradient task to the weight-gradient task.  ``JAXPP_B200_ZB_DEFER_BYTES`` bounds those bytes by running
    the weight gradients that do not fit with the activation gradients; results do not change."""
    import math

    from jaxpp_b200.compiler.program import RunTask
    from jaxpp_b200.utils import config

    sched = jp.ZeroBubble(2)
    cfg = tf.ModelConfig("llama", vocab=128, d_model=32, n_layers=2, n_heads=2, n_kv_heads=2, ffn=64, seq=16, n_stages=2,
                         dtype=torch.float32, recompute=True)
    step = lt.make_train_step(cfg, sched, lt.Hyper(lr=1e-2, inplace_update=False))
    state = lt.init_state(cfg, sched, "cpu")
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, 128, (4, 2, 16), generator=g)
    labels = torch.randint(0, 128, (4, 2, 16), generator=g)
    ref = step(state, tokens, labels)

    def carried(prog):
        a = next(i for i in prog.instrs if isinstance(i, RunTask) and i.name == "bwdA_1__0")
        w = next(i for i in prog.instrs if isinstance(i, RunTask) and i.name == "bwdW_1__0")
        vids = set(a.outs) & set(w.ins)
        wgrads = sum("linear_wgrad" in str(t) for t in w.code.targets)
        return sum(math.prod(prog.values[v].shape) * prog.values[v].dtype.itemsize for v in vids), wgrads

    seen = {}
    for budget in (-1, 40000, 0):
        with config.zb_defer_bytes.set(budget):
            f = jp.mpmd_jit_with_loop(step, cpu_mesh(2))
            prog = f.lower(state, tokens, labels).program
            got = f(state, tokens, labels)
        assert_trees_equal(ref, got, exact=True)
        seen[budget] = carried(prog)
    assert seen[-1][0] > seen[40000][0] > seen[0][0] == 0
    assert seen[40000][0] <= 40000 and seen[-1][1] == 1 and seen[0][1] == 0
