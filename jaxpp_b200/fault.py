"""Failure detection and host-side fault injection.

The reference only has coordinator time-outs (``heartbeat_timeout_seconds=5`` etc.,
src/jaxpp/distributed_utils.py:26-33) and a fail-fast launcher.  Here every process runs a heartbeat thread
that publishes ``(step, wall time)`` in the rendezvous key-value store and a watchdog that reads its peers':

* a peer whose heartbeat is older than the time-out, or that published a failure record, makes
  :meth:`FailureDetector.check` raise :class:`PeerFailure` on every other rank *before their next launch* —
  so nobody enqueues a collective that can never complete;
* a step that runs past its deadline is reported by the step watchdog;
* recovery is restart-from-checkpoint (the launcher exits non-zero; see ``checkpoint.latest_step``).

Faults are injected on the host only: an exception in a named task, a dropped or delayed transfer, a rank that
stops heart-beating.  Device-side waits are bounded separately and report through the kernel status word.
"""
from __future__ import annotations

import contextlib
import dataclasses
import json
import threading
import time
from typing import Callable


class PeerFailure(RuntimeError):
    """Another rank failed or stopped responding."""


class StepTimeout(RuntimeError):
    pass


class InjectedFault(RuntimeError):
    pass


class DictStore:
    """In-process stand-in for the rendezvous store (tests, single-process runs)."""

    def __init__(self):
        self._d: dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value):
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d[key]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


def default_store():
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.distributed_c10d._get_default_store()
    return DictStore()


class FailureDetector:
    def __init__(self, rank: int, world: int, store=None, interval_s: float = 0.5, timeout_s: float = 5.0,
                 prefix: str = "jaxpp_b200/hb", clock: Callable[[], float] = time.time):
        self.rank, self.world = rank, world
        self.store = store if store is not None else default_store()
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self.prefix = prefix
        self.clock = clock
        self.step = 0
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._thread: threading.Thread | None = None
        self._failed_peer: tuple[int, str] | None = None
        self._step_deadline: float | None = None
        self._first_seen: dict[int, float] = {}

    # -- heartbeat --------------------------------------------------------------------------------------
    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self):
        self.store.set(self._key(self.rank), json.dumps({"step": self.step, "t": self.clock(), "ok": True}))

    def report_failure(self, reason: str):
        """Publish that this rank is going down (called from exception handlers)."""
        try:
            self.store.set(self._key(self.rank), json.dumps({"step": self.step, "t": self.clock(), "ok": False,
                                                             "reason": reason[:500]}))
        except Exception:
            pass

    def _loop(self):
        while not self._stop.wait(self.interval_s):
            if not self._paused.is_set():
                try:
                    self.beat()
                except Exception:
                    return
            self._scan()

    def start(self):
        self.beat()
        self._thread = threading.Thread(target=self._loop, name="jaxpp-b200-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)

    def pause_heartbeat(self, paused: bool = True):
        """Fault injection: stop publishing heartbeats while staying alive."""
        (self._paused.set if paused else self._paused.clear)()

    # -- watchdog -------------------------------------------------------------------------------------------
    def _scan(self):
        now = self.clock()
        for r in range(self.world):
            if r == self.rank or self._failed_peer is not None:
                continue
            key = self._key(r)
            try:
                if not self.store.check([key]):
                    first = self._first_seen.setdefault(r, now)
                    if now - first > max(self.timeout_s * 4, 20.0):
                        self._failed_peer = (r, "never published a heartbeat")
                    continue
                rec = json.loads(self.store.get(key))
            except Exception as e:  # the store itself is gone: rank 0 (its host) died
                self._failed_peer = (0, f"rendezvous store unreachable: {e}")
                return
            if not rec.get("ok", True):
                self._failed_peer = (r, rec.get("reason", "reported failure"))
            elif now - rec["t"] > self.timeout_s:
                self._failed_peer = (r, f"no heartbeat for {now - rec['t']:.1f}s (last at step {rec['step']})")
        if self._step_deadline is not None and now > self._step_deadline and self._failed_peer is None:
            self._failed_peer = (self.rank, f"step {self.step} exceeded its deadline")

    def check(self):
        """Raise if a peer has failed.  Call between steps / before launching work that needs the peers."""
        self._scan()
        if self._failed_peer is not None:
            r, why = self._failed_peer
            if r == self.rank:
                raise StepTimeout(why)
            raise PeerFailure(f"pipeline peer {r} failed: {why}")

    @contextlib.contextmanager
    def step_scope(self, step: int, deadline_s: float | None = None):
        self.step = step
        self._step_deadline = self.clock() + deadline_s if deadline_s else None
        try:
            yield
        except BaseException as e:
            self.report_failure(f"{type(e).__name__}: {e}")
            raise
        finally:
            self._step_deadline = None


# ---- host-side fault injection -----------------------------------------------------------------------------
@dataclasses.dataclass
class FaultPlan:
    """What to break, where: all fields are matched on the host."""

    raise_in_task: str | None = None   # task name prefix, e.g. "bwd_1__2"
    on_rank: int | None = None
    at_step: int | None = None
    drop_transfer: int | None = None   # transfer id never sent
    delay_transfer_s: float = 0.0


_PLAN: list[FaultPlan | None] = [None]
_STEP = [0]


def set_fault_plan(plan: FaultPlan | None):
    _PLAN[0] = plan


def set_current_step(step: int):
    _STEP[0] = step


def maybe_fail_task(rank: int, task_name: str):
    plan = _PLAN[0]
    if plan is None or plan.raise_in_task is None:
        return
    if plan.on_rank is not None and plan.on_rank != rank:
        return
    if plan.at_step is not None and plan.at_step != _STEP[0]:
        return
    if task_name.startswith(plan.raise_in_task):
        raise InjectedFault(f"injected failure in task {task_name} on rank {rank}")


def transfer_action(rank: int, tid: int) -> str:
    """'send', 'drop' or 'delay' for a transfer this rank is about to send."""
    plan = _PLAN[0]
    if plan is None or (plan.on_rank is not None and plan.on_rank != rank):
        return "send"
    if plan.at_step is not None and plan.at_step != _STEP[0]:
        return "send"
    if plan.drop_transfer == tid:
        return "drop"
    if plan.delay_transfer_s > 0:
        time.sleep(plan.delay_transfer_s)
        return "delay"
    return "send"
