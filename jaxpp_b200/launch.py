"""Process bootstrap and a single-node multi-process launcher.

Counterpart of the reference's ``distributed_main`` / ``JaxDistributedTest``
(src/jaxpp/distributed_utils.py:25-55) and of its launcher script (scripts/local_mc.sh:46-82): N worker
processes on one node, rendezvous on 127.0.0.1, fail fast — when any worker exits non-zero the others
are terminated (their process groups, not a name pattern) and the launcher reports which rank failed.
"""
from __future__ import annotations

import datetime
import os
import signal
import socket
import subprocess
import sys
import time
from typing import Callable, Sequence


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def distributed_main(fn: Callable[[], None], backend: str | None = None, timeout_s: float = 120.0) -> None:
    """Initialise ``torch.distributed`` from the ``RANK``/``WORLD_SIZE``/``MASTER_*`` environment, run ``fn``,
    tear down.  ``backend`` defaults to nccl when CUDA is available, else gloo."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1:
        return fn()
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kw = {}
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    try:
        fn()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def launch(argv: Sequence[str], nproc: int, env: dict | None = None, timeout_s: float = 600.0,
           gpus_per_proc: int = 0) -> int:
    """Run ``python argv...`` as ``nproc`` ranks.  Returns 0 if all exit 0, else the first failing code.

    With ``gpus_per_proc > 0`` rank ``i`` sees only its own slice of the node's GPUs.
    """
    port = free_port()
    procs: list[subprocess.Popen] = []
    for rank in range(nproc):
        e = dict(os.environ)
        e.update(env or {})
        e.update({"RANK": str(rank), "WORLD_SIZE": str(nproc), "LOCAL_RANK": str(rank), "LOCAL_WORLD_SIZE": str(nproc),
                  "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
        if gpus_per_proc > 0:
            first = rank * gpus_per_proc
            e["CUDA_VISIBLE_DEVICES"] = ",".join(str(first + k) for k in range(gpus_per_proc))
            e["LOCAL_RANK"] = "0"
        procs.append(subprocess.Popen([sys.executable, *argv], env=e, start_new_session=True))
    deadline = time.time() + timeout_s
    rc = 0
    try:
        while True:
            codes = [p.poll() for p in procs]
            failed = [(i, c) for i, c in enumerate(codes) if c not in (None, 0)]
            if failed:
                rc = failed[0][1]
                sys.stderr.write(f"[launch] rank {failed[0][0]} exited with {rc}; stopping the others\n")
                break
            if all(c == 0 for c in codes):
                return 0
            if time.time() > deadline:
                sys.stderr.write("[launch] timeout; stopping all ranks\n")
                rc = 124
                break
            time.sleep(0.05)
    finally:
        for p in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)  # the worker's own process group
                except ProcessLookupError:
                    pass
        for p in procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
    return rc


def _main(args: list[str]) -> int:
    """``launch.py --nproc N [--timeout S] (script.py | -m module) [args of the script ...]``: everything after
    the script or module name goes to the workers untouched."""
    nproc, timeout_s, i = None, 600.0, 0
    while i < len(args):
        if args[i] == "--nproc":
            nproc, i = int(args[i + 1]), i + 2
        elif args[i] == "--timeout":
            timeout_s, i = float(args[i + 1]), i + 2
        else:
            break
    rest = args[i:]
    if nproc is None or not rest or (rest[0] == "-m" and len(rest) < 2):
        sys.stderr.write("usage: python -m jaxpp_b200.launch --nproc N [--timeout S] (script.py | -m module) [args ...]\n")
        return 2
    return launch(rest, nproc, timeout_s=timeout_s)


if __name__ == "__main__":
    sys.exit(_main(sys.argv[1:]))
