"""Failure detection without touching a GPU: heartbeats over a store, host-side fault injection among
CPU (gloo) ranks, bounded detection time."""
import os
import threading
import time

import pytest

from jaxpp_b200 import fault
from jaxpp_b200.launch import launch

HERE = os.path.dirname(os.path.abspath(__file__))


def test_detector_sees_stale_and_failed_peers():
    store = fault.DictStore()
    now = [100.0]
    a = fault.FailureDetector(0, 3, store, timeout_s=2.0, clock=lambda: now[0])
    b = fault.FailureDetector(1, 3, store, timeout_s=2.0, clock=lambda: now[0])
    c = fault.FailureDetector(2, 3, store, timeout_s=2.0, clock=lambda: now[0])
    for d in (a, b, c):
        d.beat()
    a.check()
    now[0] += 1.0
    a.beat(), b.beat()          # rank 2 goes silent
    a.check()
    now[0] += 1.5
    a.beat(), b.beat()
    with pytest.raises(fault.PeerFailure, match="peer 2 failed: no heartbeat"):
        a.check()
    # an explicit failure report is seen at once
    store2 = fault.DictStore()
    x = fault.FailureDetector(0, 2, store2, timeout_s=50.0)
    y = fault.FailureDetector(1, 2, store2, timeout_s=50.0)
    x.beat(), y.beat()
    with pytest.raises(ValueError):
        with y.step_scope(7):
            raise ValueError("boom")
    with pytest.raises(fault.PeerFailure, match="ValueError: boom"):
        x.check()


def test_step_deadline():
    now = [0.0]
    d = fault.FailureDetector(0, 1, fault.DictStore(), clock=lambda: now[0])
    with d.step_scope(1, deadline_s=5.0):
        now[0] = 4.0
        d.check()
        now[0] = 6.0
        with pytest.raises(fault.StepTimeout, match="step 1 exceeded"):
            d.check()


def test_heartbeat_thread_and_pause():
    store = fault.DictStore()
    a = fault.FailureDetector(0, 2, store, interval_s=0.05, timeout_s=0.4).start()
    b = fault.FailureDetector(1, 2, store, interval_s=0.05, timeout_s=0.4).start()
    try:
        time.sleep(0.3)
        a.check(), b.check()
        b.pause_heartbeat()
        deadline = time.time() + 3.0
        seen = False
        while time.time() < deadline and not seen:
            try:
                a.check()
                time.sleep(0.05)
            except fault.PeerFailure:
                seen = True
        assert seen, "a silent peer was not detected within the deadline"
    finally:
        a.stop(), b.stop()


def test_launcher_fail_fast():
    """One rank exits non-zero: the launcher stops the others and reports the failing code quickly."""
    script = os.path.join(HERE, "fault_worker.py")
    t0 = time.time()
    rc = launch([script, "exit_early"], 3, env={"CUDA_VISIBLE_DEVICES": ""}, timeout_s=120)
    assert rc == 7 and time.time() - t0 < 60


@pytest.mark.parametrize("mode", ["raise_in_task", "drop_transfer", "silent_rank"])
def test_injected_faults_among_cpu_ranks(mode):
    """A pipeline of gloo ranks: one rank fails (exception in a task, a dropped message, or it goes silent);
    every surviving rank must notice through the failure detector and exit with the dedicated code."""
    script = os.path.join(HERE, "fault_worker.py")
    rc = launch([script, mode], 2, env={"CUDA_VISIBLE_DEVICES": "", "OMP_NUM_THREADS": "1"}, timeout_s=120)
    assert rc in (41, 42), f"unexpected exit code {rc}"
