"""Worker for tests/test_fault.py (CPU ranks over gloo)."""
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

mode = sys.argv[1]
rank = int(os.environ["RANK"])

if mode == "exit_early":
    if rank == 1:
        sys.exit(7)
    time.sleep(60)
    sys.exit(0)

import datetime  # noqa: E402

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import jaxpp_b200 as jp  # noqa: E402
from jaxpp_b200 import fault  # noqa: E402

from helpers import make_mlp_step, mlp_params  # noqa: E402

EXIT_SAW_PEER_FAILURE = 41   # a healthy rank learned of the failure and left cleanly
EXIT_INJECTED = 42           # the rank on which the fault was injected

dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
world = dist.get_world_size()
det = fault.FailureDetector(rank, world, interval_s=0.1, timeout_s=1.5).start()
mesh = jp.MpmdMesh.create({"mpmd": world, "data": 1, "model": 1}, kind="cpu", multi_process=True)
sched = jp.Std1F1B(world)
step = make_mlp_step(world, sched, 4)
f = jp.mpmd_jit_with_loop(step, mesh)
params, batch = mlp_params(world, 16), torch.randn(4, 4, 16)


def watchdog_exit():
    # the main thread may be blocked inside a receive that can never complete: the watchdog thread ends the
    # process as soon as the detector knows a peer is gone
    while True:
        time.sleep(0.1)
        try:
            det.check()
        except fault.PeerFailure as e:
            print(f"[rank {rank}] {e}", flush=True)
            os._exit(EXIT_SAW_PEER_FAILURE)
        except fault.StepTimeout:
            os._exit(EXIT_SAW_PEER_FAILURE)


threading.Thread(target=watchdog_exit, daemon=True).start()

out = f(params, batch)  # step 0: healthy
for s in range(1, 4):
    fault.set_current_step(s)
    if mode == "raise_in_task":
        fault.set_fault_plan(fault.FaultPlan(raise_in_task="bwd_1", on_rank=1, at_step=2))
    elif mode == "drop_transfer":
        fault.set_fault_plan(fault.FaultPlan(drop_transfer=2, on_rank=1, at_step=2))
    elif mode == "silent_rank" and s == 2 and rank == 1:
        det.pause_heartbeat()
        time.sleep(30)  # alive but unresponsive; peers must not wait for it
        os._exit(EXIT_INJECTED)
    try:
        with det.step_scope(s, deadline_s=5.0):
            det.check()
            out = f(out[1], batch)
    except fault.InjectedFault as e:
        print(f"[rank {rank}] {e}", flush=True)
        time.sleep(0.5)  # let the failure record reach the store
        os._exit(EXIT_INJECTED)
    except fault.PeerFailure as e:
        print(f"[rank {rank}] {e}", flush=True)
        os._exit(EXIT_SAW_PEER_FAILURE)
print(f"[rank {rank}] finished without noticing the fault", flush=True)
os._exit(3)
