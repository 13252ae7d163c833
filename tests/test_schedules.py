"""Schedules: per-rank task orders, validation errors, stage→rank maps, dependency replay."""
import pytest

from jaxpp_b200.schedules import (DualPipeV, Eager1F1B, FusedTask, GPipe, Interleaved1F1B, InterleavedGPipe, KimiK2,
                                  Std1F1B, ZeroBubble, preprocess_schedule_tasks, replay)
from jaxpp_b200.types import TaskType


def names(schedule, n, unpack=False):
    return [[str(t) for t in r] for r in preprocess_schedule_tasks(schedule.tasks(n), 0, unpack)]


def short(seq):
    """f0 b1 A2 W3 notation for single-stage-per-rank schedules."""
    m = {"fwd": "f", "bwd": "b", "bwdA": "A", "bwdW": "W"}
    return " ".join(m[s.split("_")[0]] + s.split("__")[1] for s in seq)


def test_std1f1b_golden():
    assert names(Std1F1B(2), 4) == [
        "fwd_0__0 fwd_0__1 bwd_0__0 fwd_0__2 bwd_0__1 fwd_0__3 bwd_0__2 bwd_0__3".split(),
        "fwd_1__0 bwd_1__0 fwd_1__1 bwd_1__1 fwd_1__2 bwd_1__2 fwd_1__3 bwd_1__3".split(),
    ]
    got = [short(r) for r in names(Std1F1B(4), 8)]
    assert got[0] == "f0 f1 f2 f3 b0 f4 b1 f5 b2 f6 b3 f7 b4 b5 b6 b7"
    assert got[1] == "f0 f1 f2 b0 f3 b1 f4 b2 f5 b3 f6 b4 f7 b5 b6 b7"
    assert got[2] == "f0 f1 b0 f2 b1 f3 b2 f4 b3 f5 b4 f6 b5 f7 b6 b7"
    assert got[3] == " ".join(f"f{i} b{i}" for i in range(8))


def test_eager1f1b_and_gpipe_golden():
    got = [short(r) for r in names(Eager1F1B(3), 5)]
    assert got == ["f0 f1 f2 f3 f4 b0 b1 b2 b3 b4", "f0 f1 f2 b0 f3 b1 f4 b2 b3 b4", "f0 b0 f1 b1 f2 b2 f3 b3 f4 b4"]
    assert [short(r) for r in names(GPipe(2), 3)] == ["f0 f1 f2 b0 b1 b2"] * 2


def test_zero_bubble_golden():
    got = [short(r) for r in names(ZeroBubble(4), 4)]
    assert got[0] == "f0 f1 f2 f3 A0 A1 A2 A3"  # first stage: halves merged into one task typed BWD_I
    assert got[1] == "f0 f1 f2 A0 f3 A1 W0 A2 W1 A3 W2 W3"
    assert got[2] == "f0 f1 A0 f2 A1 f3 A2 W0 A3 W1 W2 W3"
    assert got[3] == "f0 A0 f1 A1 f2 A2 f3 A3 W0 W1 W2 W3"
    r1 = short(names(ZeroBubble(4), 8)[1])
    assert r1 == "f0 f1 f2 A0 f3 A1 W0 f4 A2 W1 f5 A3 W2 f6 A4 W3 f7 A5 W4 A6 W5 A7 W6 W7"
    merged = preprocess_schedule_tasks(ZeroBubble(4).tasks(4), 0, False)[0]
    assert all(t.latency == 2 for t in merged if t.fwd_or_bwd is TaskType.BWD_I)
    with pytest.raises(AssertionError, match="Expect num of microbatches >= num of stages"):
        ZeroBubble(4).tasks(3)


def test_interleaved_golden():
    r0, r1 = names(Interleaved1F1B(num_stages=4, mpmd_dim=2), 4)
    assert r0 == ("fwd_0__0 fwd_0__1 fwd_2__0 fwd_2__1 fwd_0__2 bwd_2__0 fwd_0__3 bwd_2__1 fwd_2__2 bwd_0__0 "
                  "fwd_2__3 bwd_0__1 bwd_2__2 bwd_2__3 bwd_0__2 bwd_0__3").split()
    assert r1 == ["fwd_1__0", "fwd_1__1", "FusedTask(fwd_3__0, bwd_3__0)", "FusedTask(fwd_3__1, bwd_3__1)",
                  "fwd_1__2", "bwd_1__0", "fwd_1__3", "bwd_1__1", "FusedTask(fwd_3__2, bwd_3__2)",
                  "FusedTask(fwd_3__3, bwd_3__3)", "bwd_1__2", "bwd_1__3"]
    r = names(Interleaved1F1B(8, 4), 8)
    exp0 = ([f"fwd_0__{m}" for m in range(4)] + [f"fwd_4__{m}" for m in range(4)]
            + "fwd_0__4 fwd_0__5 fwd_0__6 bwd_4__0 fwd_0__7 bwd_4__1 fwd_4__4 bwd_4__2 fwd_4__5 bwd_4__3 fwd_4__6 "
              "bwd_0__0 fwd_4__7 bwd_0__1 bwd_0__2 bwd_0__3".split()
            + [f"bwd_4__{m}" for m in range(4, 8)] + [f"bwd_0__{m}" for m in range(4, 8)])
    assert r[0] == exp0
    exp3 = ([f"fwd_3__{m}" for m in range(4)] + [f"FusedTask(fwd_7__{m}, bwd_7__{m})" for m in range(4)]
            + "fwd_3__4 bwd_3__0 fwd_3__5 bwd_3__1 fwd_3__6 bwd_3__2 fwd_3__7 bwd_3__3".split()
            + [f"FusedTask(fwd_7__{m}, bwd_7__{m})" for m in range(4, 8)] + [f"bwd_3__{m}" for m in range(4, 8)])
    assert r[3] == exp3
    # with as many stages as ranks it degenerates to plain 1F1B
    assert names(Interleaved1F1B(4, 4), 4, unpack=True)[2] == \
        "fwd_2__0 fwd_2__1 fwd_2__2 bwd_2__0 fwd_2__3 bwd_2__1 bwd_2__2 bwd_2__3".split()


def test_kimik2_golden():
    r0 = names(KimiK2(8, 4, fuse_steady_state=True), 8)[0]
    exp = ([f"fwd_0__{m}" for m in range(4)] + [f"fwd_4__{m}" for m in range(4)] + ["fwd_0__4", "fwd_0__5", "fwd_0__6"]
           + ["FusedTask(fwd_0__7, bwd_4__0)", "FusedTask(fwd_4__4, bwd_4__1)", "FusedTask(fwd_4__5, bwd_4__2)",
              "FusedTask(fwd_4__6, bwd_4__3)", "FusedTask(fwd_4__7, bwd_0__0)", "bwd_0__1", "bwd_0__2", "bwd_0__3"]
           + [f"bwd_4__{m}" for m in range(4, 8)] + [f"bwd_0__{m}" for m in range(4, 8)])
    assert r0 == exp


def test_dualpipev_golden():
    r0, r1 = names(DualPipeV(num_stages=4, mpmd_dim=2), 4)
    assert r0 == ["fwd_0__0", "fwd_0__1", "fwd_0__2", "fwd_3__0", "bwdA_3__0", "bwdW_3__0", "fwd_3__1",
                  "FusedTask(fwd_0__3, bwdA_3__1, bwdW_3__1)", "FusedTask(fwd_3__2, bwdA_0__0)",
                  "FusedTask(bwdA_3__2, bwdW_3__2)", "FusedTask(fwd_3__3, bwdA_0__1)",
                  "FusedTask(bwdA_3__3, bwdW_3__3)", "bwdA_0__2", "bwdA_0__3"]
    assert r1 == ["fwd_1__0", "fwd_2__0", "fwd_1__1", "fwd_2__1", "fwd_1__2", "FusedTask(bwdA_2__0, bwdW_2__0)",
                  "FusedTask(fwd_2__2, bwdA_1__0, bwdW_1__0)", "FusedTask(fwd_1__3, bwdA_2__1, bwdW_2__1)",
                  "FusedTask(fwd_2__3, bwdA_1__1, bwdW_1__1)", "FusedTask(bwdA_2__2, bwdW_2__2)",
                  "FusedTask(bwdA_1__2, bwdW_1__2)", "bwdA_2__3", "FusedTask(bwdA_1__3, bwdW_1__3)", "bwdW_2__3"]


def test_stage_to_rank_maps():
    assert [Std1F1B(4).get_mpmd_idx(s) for s in range(4)] == [0, 1, 2, 3]
    assert [Interleaved1F1B(8, 4).get_mpmd_idx(s) for s in range(8)] == [0, 1, 2, 3, 0, 1, 2, 3]
    assert [DualPipeV(8, 4).get_mpmd_idx(s) for s in range(8)] == [0, 1, 2, 3, 3, 2, 1, 0]


@pytest.mark.parametrize("schedule,n", [
    (Std1F1B(4), 8), (Eager1F1B(4), 8), (GPipe(3), 5), (ZeroBubble(4), 6), (Interleaved1F1B(8, 4), 8),
    (KimiK2(8, 4), 8), (InterleavedGPipe(8, 4), 8), (DualPipeV(8, 4), 10), (Interleaved1F1B(6, 3, True), 6),
])
def test_list_lengths_and_coverage(schedule, n):
    lists = schedule.tasks(n)
    assert len(lists) == schedule.num_ranks
    flat = [t for r in preprocess_schedule_tasks(lists, 0, True) for t in r]
    keys = {(t.stage_id, t.mubatch_idx, t.fwd_or_bwd) for t in flat}
    assert len(keys) == len(flat)  # nothing runs twice
    fwd = {(s, m) for s, m, k in keys if k is TaskType.FWD}
    assert fwd == {(s, m) for s in range(schedule.num_stages) for m in range(n)}
    makespan, busy, _ = replay(schedule, n)  # raises if the orders deadlock
    assert makespan >= max(busy)


def test_validation_messages():
    with pytest.raises(ValueError, match="The argument `num_stages` must be `>= 0`"):
        Std1F1B(0)
    with pytest.raises(ValueError, match="The argument `mpmd_dim` must be `>= 0`"):
        Interleaved1F1B(4, 0)
    with pytest.raises(ValueError, match="can not be evenly divided by"):
        Interleaved1F1B(5, 2)
    with pytest.raises(ValueError, match="DualPipeV only supports 2 \\* mpmd_dim stages, self.num_stages=6 requested with self.mpmd_dim=2"):
        DualPipeV(6, 2)
    with pytest.raises(ValueError, match="DualPipeV requires n_mubatches=3 >= self.num_stages=4"):
        DualPipeV(4, 2).tasks(3)
    with pytest.raises(ValueError, match="n_microbatches must be divisible by mpmd_dim"):
        Interleaved1F1B(4, 2).tasks(5)


def test_ideal_bubbles():
    assert Std1F1B(2).ideal_bubble_fraction(16) == pytest.approx(1 / 17)
    assert Interleaved1F1B(8, 4).ideal_bubble_fraction(32) == pytest.approx(3 / 67)
    assert ZeroBubble(4).ideal_bubble_fraction(64) < Std1F1B(4).ideal_bubble_fraction(64)


def test_fused_task_properties():
    t = Interleaved1F1B(4, 2).tasks(4)[1][2]
    assert isinstance(t, FusedTask) and t.latency == 3
