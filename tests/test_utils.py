"""Flag classes and small utilities (behaviour of the reference's tests/test_utils.py)."""
import logging
import os

import pytest

from jaxpp_b200.utils import (BoolEnvVar, IntEnvVar, OverwriteableVar, StrEnvVar, format_bytes, groupby, hbytes,
                              log_elapsed_time, parse_bool, partition, unzip_multi)


def test_unzip_multi():
    assert unzip_multi([(1, "a"), (2, "b")]) == [[1, 2], ["a", "b"]]
    assert unzip_multi([], arity=3) == [[], [], []]
    assert unzip_multi([(1, 2, 3)], arity=3) == [[1], [2], [3]]
    with pytest.raises(AssertionError):
        unzip_multi([(1, 2), (3,)])


def test_groupby_partition():
    assert groupby([("a", 1), ("b", 2), ("a", 3)]) == {"a": [1, 3], "b": [2]}
    assert partition(lambda x: x % 2 == 0, range(5)) == ([0, 2, 4], [1, 3])


def test_log_elapsed_time(caplog):
    log = logging.getLogger("t")
    with caplog.at_level(logging.INFO, logger="t"):
        with log_elapsed_time("evt", msg="hello", log=log):
            pass
        with log_elapsed_time("evt2", unit="ms", log=log):
            pass
    assert "[evt] hello took" in caplog.text and caplog.text.count("ms") >= 1
    with pytest.raises(ValueError, match="Unknown unit"):
        with log_elapsed_time("evt", unit="h"):
            pass


def test_overwriteable_var():
    v = OverwriteableVar(3)
    assert v.value == 3
    with v.set(5):
        assert v.value == 5
        with v.set(7):
            assert v.value == 7
        assert v.value == 5
    assert v.value == 3
    with pytest.raises(ValueError, match="truthy"):
        bool(v)


def test_parse_bool():
    for s in ["true", "1", "T", "y", "YES"]:
        assert parse_bool(s) is True
    for s in ["false", "0", "F", "n", "No"]:
        assert parse_bool(s) is False
    assert parse_bool("maybe") is None


def test_env_vars(monkeypatch):
    monkeypatch.setenv("X_BOOL", "yes")
    monkeypatch.setenv("X_INT", "12")
    monkeypatch.setenv("X_STR", "abc")
    monkeypatch.setenv("X_BAD", "twelve")
    assert BoolEnvVar("X_BOOL", False).value is True
    assert IntEnvVar("X_INT", 1).value == 12
    assert StrEnvVar("X_STR", "").value == "abc"
    assert BoolEnvVar("X_MISSING", True).value is True
    with pytest.raises(ValueError, match="Unsupported value X_BAD=twelve"):
        IntEnvVar("X_BAD", 0).value
    # the environment is read once
    v = IntEnvVar("X_INT", 1)
    assert v.value == 12
    monkeypatch.setenv("X_INT", "13")
    assert v.value == 12
    with v.set(99):
        assert v.value == 99
    assert v.value == 12


def test_bytes():
    assert format_bytes(512) == "512B"
    assert format_bytes(2048) == "2.00KiB"
    assert hbytes([1024 * 1024, 1024 * 1024]) == "2.00MiB"


def test_dropout_is_a_pure_function_of_seed_offset_and_index():
    import torch

    from jaxpp_b200.ops import core as ops

    # known answer of Philox4x32-10 for the all-zero counter and key (Random123 test vectors)
    w = ops.philox_u32(1, torch.tensor(0), 0, "cpu")[0]
    assert [int(v) for v in w] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    x = torch.ones(3, 1001)
    seed = torch.tensor(99, dtype=torch.int64)
    y = ops.dropout(x, 0.25, seed, 5)
    assert torch.equal(y, ops.dropout(x, 0.25, seed, 5))
    assert not torch.equal(y, ops.dropout(x, 0.25, seed, 6))
    assert not torch.equal(y, ops.dropout(x, 0.25, seed + 1, 5))
    assert abs((y == 0).float().mean().item() - 0.25) < 0.03 and torch.allclose(y[y != 0], torch.tensor(1 / 0.75))
    xr = x.clone().requires_grad_(True)
    (g,) = torch.autograd.grad(ops.dropout(xr, 0.25, seed, 5).sum(), [xr])
    assert torch.equal(g, y)  # backward regenerates the same mask


def test_launcher_cli_runs_modules_and_passes_arguments_through(tmp_path):
    """``python -m jaxpp_b200.launch --nproc N (script | -m module) args...``: everything after the script or module
    name reaches the workers untouched, every rank gets its rendezvous environment, a failing rank fails the launch."""
    import subprocess
    import sys

    script = tmp_path / "worker.py"
    script.write_text(
        "import os, sys\n"
        "out = os.path.join(sys.argv[2], 'rank%s.txt' % os.environ['RANK'])\n"
        "open(out, 'w').write(' '.join(sys.argv[1:]) + ' ' + os.environ['WORLD_SIZE'] + ' ' + os.environ['MASTER_ADDR'])\n"
        "sys.exit(3 if sys.argv[1] == '--fail' and os.environ['RANK'] == '1' else 0)\n")
    cmd = [sys.executable, "-m", "jaxpp_b200.launch", "--nproc", "2", "--timeout", "60", str(script)]
    ok = subprocess.run(cmd + ["--iters", str(tmp_path), "--flag"], capture_output=True, text=True)
    assert ok.returncode == 0, ok.stderr
    for r in (0, 1):
        assert (tmp_path / f"rank{r}.txt").read_text() == f"--iters {tmp_path} --flag 2 127.0.0.1"
    bad = subprocess.run(cmd + ["--fail", str(tmp_path)], capture_output=True, text=True)
    assert bad.returncode == 3 and "rank 1 exited with 3" in bad.stderr
    usage = subprocess.run([sys.executable, "-m", "jaxpp_b200.launch", "--nproc", "2"], capture_output=True, text=True)
    assert usage.returncode == 2 and "usage" in usage.stderr


def test_optimizer_state_slices_cover_a_parameter_exactly_once():
    """Flat 1/n slices of a parameter (``parallel/zero.py``): padded to whole 16-byte vectors for 2- and 4-byte types,
    their concatenation restores the parameter, and placeholders of other pipeline ranks get the slice shape."""
    import torch

    import jaxpp_b200 as jp
    from jaxpp_b200.parallel import zero

    for numel, n in ((1, 2), (8, 2), (17, 4), (1000003, 8), (4096 * 4096, 4)):
        s = zero.shard_numel(numel, n)
        assert s % 8 == 0 and s * n >= numel and (s - 8) * n < numel
    t = torch.arange(37.0).view(37, 1)
    parts = [zero.local_shard(t, 4, r) for r in range(4)]
    assert all(p.shape == (16,) for p in parts)
    whole = torch.cat(parts)
    assert torch.equal(whole[:37], t.view(-1)) and whole[37:].abs().sum() == 0
    state = {"params": {"w": t}, "master": {"w": t.clone(), "e": jp.ShapeDtypeStruct((5, 3), torch.float32)},
             "m": {"w": torch.zeros_like(t), "e": jp.ShapeDtypeStruct((5, 3), torch.float32)},
             "v": {"w": torch.zeros_like(t), "e": jp.ShapeDtypeStruct((5, 3), torch.float32)}, "step": torch.zeros(())}
    sharded = zero.shard_optimizer_state(state, 4, 1, keep=lambda path: False)
    assert torch.equal(sharded["master"]["w"], parts[1]) and sharded["m"]["e"].shape == (8,)
    assert sharded["params"]["w"] is t                                    # the compute copy stays whole
    kept = zero.shard_optimizer_state(state, 4, 1, keep=lambda path: path == ("w",))
    assert kept["master"]["w"].shape == (37, 1)
    # outside a mesh axis of size > 1 the ops are the identity on the padded flat tensor
    mesh = jp.MpmdMesh.create({"mpmd": 1, "data": 1, "model": 1}, kind="cpu", multi_process=False)
    with mesh:
        flat = zero.reduce_scatter_flat(t, "data", 0.5)
        assert flat.shape == (40,) and torch.equal(flat[:37], t.view(-1) * 0.5)
        assert torch.equal(zero.all_gather_flat(flat, "data", 37), t.view(-1) * 0.5)


def test_public_api_names():
    """Every name of the reference's façade (src/jaxpp/api.py:19-65) is importable from the package root and from
    ``jaxpp_b200.api``, with the call shapes its users rely on."""
    import inspect

    import jaxpp_b200 as jp
    from jaxpp_b200 import api

    names = ["mpmd_jit_with_loop", "mpmd_jit_by_yield", "treduce", "treduce_i", "Add", "Max", "Concat", "mark_stage_end",
             "pipeline_enter_stage", "MpmdMesh", "MpmdArray", "MpmdSharding", "BaseSchedule", "Std1F1B", "Eager1F1B",
             "Interleaved1F1B", "KimiK2", "ZeroBubble", "DualPipeV", "cross_mpmd_all_reduce", "cross_mpmd_stack", "place_with",
             "spmd_to_mpmd_reshard", "mpmd_to_spmd_reshard", "collect_task_times_ms", "_to_global_jax_array"]
    for n in names:
        assert hasattr(api, n), n
        assert getattr(jp, n) is getattr(api, n), n
    for jit in (jp.mpmd_jit_with_loop, jp.mpmd_jit_by_yield):
        params = inspect.signature(jit).parameters
        assert list(params)[:2] == ["fun", "mpmd_mesh"]
        for kw in ("in_shardings", "out_shardings", "static_argnums", "static_argnames", "donate_argnums", "donate_argnames",
                   "compiler_options"):
            assert params[kw].kind is inspect.Parameter.KEYWORD_ONLY, kw
    assert list(inspect.signature(jp.treduce).parameters)[:2] == ["fun", "xs"]
    assert {"schedule", "operation"} <= set(inspect.signature(jp.treduce).parameters)
    assert issubclass(jp.Std1F1B, jp.BaseSchedule) and jp.Interleaved1F1B(4, 2).num_stages == 4
    from jaxpp_b200.launch import distributed_main  # the bootstrap entry point of distributed_utils.py:51-54

    assert callable(distributed_main)


def test_collect_task_times_ms_records_every_task():
    """Inside the context every task run adds one sample under its name (reference: prim.py:704-859); outside, and
    with ``enabled=False``, nothing is recorded."""
    import torch

    import jaxpp_b200 as jp
    from helpers import make_mlp_step, mlp_params

    mesh = jp.MpmdMesh.create({"mpmd": 2, "data": 1, "model": 1}, kind="cpu", multi_process=False)
    f = jp.mpmd_jit_with_loop(make_mlp_step(2, jp.Std1F1B(2), 3), mesh)
    params, batch = mlp_params(2, 8), torch.randn(3, 2, 8)
    f(params, batch)
    with jp.collect_task_times_ms() as times:
        f(params, batch)
    fwd = [k for k in times if k.startswith("fwd")]
    bwd = [k for k in times if k.startswith("bwd")]
    assert len(fwd) == 6 and len(bwd) == 6 and all(len(v) == 1 and v[0] >= 0 for v in times.values())
    with jp.collect_task_times_ms(enabled=False) as nothing:
        f(params, batch)
    assert nothing is None


def test_live_bytes_tracker_reports_the_fullest_moment_of_a_step(monkeypatch):
    """With JAXPP_B200_TRACK_LIVE_BYTES=1 the executor records, per step, the bytes of distinct storages a rank's
    environment held at its fullest, which task came next and the largest values; without it nothing is recorded."""
    import torch

    import jaxpp_b200 as jp
    from helpers import make_mlp_step, mlp_params
    from jaxpp_b200.runtime import executor

    mesh = jp.MpmdMesh.create({"mpmd": 2, "data": 1, "model": 1}, kind="cpu", multi_process=False)
    f = jp.mpmd_jit_with_loop(make_mlp_step(2, jp.Std1F1B(2), 3), mesh)
    params, batch = mlp_params(2, 8), torch.randn(3, 2, 8)
    executor.LIVE_REPORT.clear()
    f(params, batch)
    assert not executor.LIVE_REPORT
    monkeypatch.setenv("JAXPP_B200_TRACK_LIVE_BYTES", "1")
    f(params, batch)
    assert len(executor.LIVE_REPORT) == 1
    rep = executor.LIVE_REPORT[-1]
    sizes = [b for b, _vid, _shape, _dtype in rep["all"]]
    assert rep["bytes"] == sum(sizes) > 0 and sizes == sorted(sizes, reverse=True) and rep["n_values"] == len(sizes)
    assert rep["largest"] == rep["all"][:12] and ":" in rep["before"]
    # aliases of one storage count once
    t = torch.zeros(16)
    total, items = executor._live_bytes({1: t, 2: t[:4], 3: torch.zeros(2)})
    assert total == 16 * 4 + 2 * 4 and len(items) == 2
    executor.LIVE_REPORT.clear()


def test_memstats_and_sharding_mesh_helpers(capsys):
    """``print_memstats`` is silent unless enabled and brackets the body with labelled reports; shardings are
    re-pointed at another mesh with their specs unchanged (reference: utils.py:223-268)."""
    import jaxpp_b200 as jp
    from jaxpp_b200.utils.misc import print_memstats, updated_named_sharding_mesh

    with print_memstats("quiet"):
        pass
    assert capsys.readouterr().out == ""
    with print_memstats("optimizer step", enabled=True):
        print("body")
    out = capsys.readouterr().out
    assert out.index("Before: optimizer step") < out.index("body") < out.index("After: optimizer step")
    a = jp.MpmdMesh.create({"mpmd": 1, "data": 2, "model": 1}, kind="cpu", multi_process=False).jax_mesh
    b = jp.MpmdMesh.create({"mpmd": 1, "data": 2, "model": 1}, kind="cpu", multi_process=False).jax_mesh
    moved = updated_named_sharding_mesh([jp.NamedSharding(a, jp.P("data")), None], b)
    assert moved[1] is None and moved[0].mesh is b and moved[0].spec == jp.P("data")


def test_memory_plan_of_the_benchmark_configurations():
    """Every named GPU configuration fits a 180 GB B200 by the planner's estimate; the schedule's peak of live
    activations follows the textbook values; sharding the optimizer state shrinks the replicated part only."""
    import dataclasses

    import jaxpp_b200 as jp
    from jaxpp_b200 import configs

    assert configs.peak_live_microbatches(jp.Std1F1B(4), 8) == [4, 3, 2, 1]          # warm-up depth of 1F1B
    assert configs.peak_live_microbatches(jp.GPipe(2), 6) == [6, 6]                  # everything in flight
    assert max(configs.peak_live_microbatches(jp.ZeroBubble(4), 8)) >= 4             # weight halves release later
    for name, rc in configs.CONFIGS.items():
        if name.startswith("encoder"):
            continue
        plan = configs.memory_plan(rc)
        assert plan["fits"], (name, plan["total"] / 1e9)
        parts = ("weights", "optimizer", "grads", "activations", "logits", "deferred_wgrad_operands")
        assert abs(plan["total"] - sum(plan[k] for k in parts)) < 1
    # zero-bubble with full recompute: every outstanding activation-gradient task holds the operands of its deferred
    # weight-gradient GEMMs; without the configuration's bounds (bf16 accumulators, 2 GB per task) 70B does not fit
    big = configs.get("llama70b_pp4tp2")
    assert configs.peak_deferred_weight_gradients(jp.ZeroBubble(4), 64) == [0, 2, 3, 4]
    loose = configs.memory_plan(big, grad_bytes=4, zb_defer_bytes=None)
    assert not loose["fits"] and loose["deferred_wgrad_operands"] > 40e9
    assert configs.memory_plan(big)["deferred_wgrad_operands"] == pytest.approx(4 * 2e9)
    mix = configs.get("mixtral8x7b_pp2ep4")
    assert not configs.memory_plan(dataclasses.replace(mix, recompute=False))["fits"]   # why that configuration recomputes
    gpt = configs.get("gpt2xl_pp2dp4")
    assert configs.memory_plan(gpt, shard_optimizer=True)["optimizer"] * 4 == pytest.approx(configs.memory_plan(gpt)["optimizer"])
    whole, sliced = configs.memory_plan(mix)["optimizer"], configs.memory_plan(mix, shard_optimizer=True)["optimizer"]
    assert 0.8 * whole < sliced < whole                                               # experts are not replicas


def test_reference_flags_without_an_effect_here_say_so(caplog):
    """Flags that exist for compatibility with the reference's launch scripts but cannot change anything in this
    design carry the reason, and a non-default setting is reported once at compile time."""
    import logging

    from jaxpp_b200.utils import config

    inert = [v for v in vars(config).values() if isinstance(v, config.EnvVar) and v.no_effect]
    assert {v.env_key for v in inert} == {
        "JAXPP_SHARE_DONATION", "JAXPP_ENABLE_LOCAL_PROPAGATION",
        "JAXPP_DIRECTIONAL_COMMUNICATORS", "JAXPP_DEBUG_SKIP_PROPAGATION", "JAXPP_FAST_INFER_SHARDINGS"}
    config._WARNED.clear()
    log = logging.getLogger("test_flags")
    with caplog.at_level(logging.WARNING, logger="test_flags"):
        config.warn_about_flags_without_effect(log)
        assert not caplog.records                       # defaults: nothing to report
        with config.fast_infer_shardings.set(True):
            config.warn_about_flags_without_effect(log)
            config.warn_about_flags_without_effect(log)   # once only
    assert len(caplog.records) == 1 and "JAXPP_FAST_INFER_SHARDINGS" in caplog.records[0].getMessage()
    config._WARNED.clear()
