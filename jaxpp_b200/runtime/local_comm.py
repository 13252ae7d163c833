"""Per-rank programs inside one process: every pipeline rank runs its own instruction list in a thread and the ranks
exchange tensors through in-process queues.

This is what ``JAXPP_DEBUG_FORCE_MPMDIFY`` selects (reference: src/jaxpp/mesh.py:124-130, src/jaxpp/core.py:3817-3820,
used by its version-matrix runs to exercise the per-process code path without launching processes): the same
``run_multi_controller`` interpreter, the same send / recv / send_done / collective instructions and the same
per-rank ordering as a one-process-per-device launch, with :class:`ThreadComm` in place of the NCCL / gloo
communicator.  A rank that fails releases the others, which then fail with a message naming it.
"""
from __future__ import annotations

import threading
from typing import Iterable, Sequence

import torch

from ..compiler.program import AllGather, Program, SendDone, Transfer
from .executor import run_multi_controller

_POLL_S = 0.05
_DEADLINE_S = 120.0


class _Hub:
    """What the ranks of one step share: message slots and collective meeting points."""

    def __init__(self, n_ranks: int):
        self.n_ranks = n_ranks
        self.cv = threading.Condition()
        self.messages: dict = {}      # (src, dst, tid) -> list of tensors
        self.meetings: dict = {}      # key -> {rank: contribution}
        self.failed: str | None = None

    def fail(self, why: str):
        with self.cv:
            if self.failed is None:
                self.failed = why
            self.cv.notify_all()

    def _wait(self, ready, what: str):
        waited = 0.0
        while not ready():
            if self.failed is not None:
                raise RuntimeError(f"another pipeline rank failed while this one waited for {what}: {self.failed}")
            if waited > _DEADLINE_S:
                raise TimeoutError(f"no partner for {what} after {_DEADLINE_S:.0f} s (mismatched per-rank programs?)")
            self.cv.wait(_POLL_S)
            waited += _POLL_S

    def put(self, key, tensors):
        with self.cv:
            self.messages[key] = tensors
            self.cv.notify_all()

    def take(self, key):
        with self.cv:
            self._wait(lambda: key in self.messages, f"transfer {key}")
            return self.messages.pop(key)

    def meet(self, key, rank: int, n: int, contribution):
        """Every one of ``n`` ranks brings a contribution; all of them get the complete ``{rank: contribution}``."""
        with self.cv:
            slot = self.meetings.setdefault(key, {"parts": {}, "left": n})
            slot["parts"][rank] = contribution
            self.cv.notify_all()
            self._wait(lambda: len(slot["parts"]) == n, f"collective {key}")
            parts = slot["parts"]
            slot["left"] -= 1
            if slot["left"] == 0:
                del self.meetings[key]
            return parts


class ThreadComm:
    """The communicator interface of :func:`~.executor.run_multi_controller` over a :class:`_Hub`."""

    def __init__(self, hub: _Hub, rank: int, device: torch.device):
        self.hub, self.rank, self.device = hub, rank, device
        self.pending: dict[int, tuple] = {}     # vid -> (message key, position in the message)
        self.fetched: dict = {}                 # message key -> tensors
        self.seq: dict[tuple, int] = {}

    def begin_step(self, st):
        self.pending.clear()
        self.fetched.clear()

    def end_step(self, st):
        self.before_use(st, list(self.pending))

    def send(self, st, ins: Transfer, prog: Program):
        self.hub.put((ins.rank, ins.dst, ins.tid), [st.env[v] for v in ins.vids])

    def recv(self, st, ins: Transfer, prog: Program):
        # posted, not waited for: like an asynchronous receive, it completes when a task first needs the value
        key = (ins.rank, ins.dst, ins.tid)
        for k, v in enumerate(ins.vids):
            self.pending[v] = (key, k)

    def before_use(self, st, vids: Iterable[int]):
        for v in vids:
            item = self.pending.pop(v, None)
            if item is None:
                continue
            key, k = item
            if key not in self.fetched:
                self.fetched[key] = self.hub.take(key)
            t = self.fetched[key][k]
            st.env[v] = t if t.device == self.device else t.to(self.device)

    def send_done(self, st, ins: SendDone):
        pass   # the receiver holds its own reference; nothing to wait for

    def all_reduce(self, buf: torch.Tensor, ranks: Sequence[int]):
        key = ("ar", tuple(ranks))
        n = self.seq[key] = self.seq.get(key, 0) + 1
        parts = self.hub.meet(key + (n,), self.rank, len(ranks), buf)
        total = None
        for r in sorted(parts):               # same order on every rank: identical results
            p = parts[r].to(self.device)
            total = p.clone() if total is None else total.add_(p)
        return total

    def all_gather(self, st, ins: AllGather, prog: Program):
        mine = {p: st.env[v] for p, v in ins.local.items()}
        parts = self.hub.meet(("ag", ins.cid), self.rank, len(ins.ranks), mine)
        merged: dict[int, torch.Tensor] = {}
        for contribution in parts.values():
            merged.update(contribution)
        return torch.cat([merged[p].to(self.device) for p in sorted(merged)], dim=ins.axis)


def run_scalarized_in_threads(prog: Program, inputs: Sequence, devices: Sequence[torch.device],
                              record_events: bool = False):
    """Run ``prog`` as ``n_ranks`` per-rank programs in threads of this process.  ``inputs[i]`` is the full flat input
    ``i``.  Returns ``(rank states, outputs)`` in the form of :func:`~.executor.run_single_controller`."""
    n = prog.n_ranks
    hub = _Hub(n)
    results: list = [None] * n
    errors: list = [None] * n

    def work(rank: int):
        try:
            dev = devices[rank]
            local = [None if x is None else (x if x.device == dev else x.to(dev)) for x in inputs]
            results[rank] = run_multi_controller(prog, rank, local, dev, ThreadComm(hub, rank, dev), record_events)
        except BaseException as e:  # noqa: BLE001 - reported to the caller below
            errors[rank] = e
            hub.fail(f"rank {rank}: {type(e).__name__}: {e}")

    threads = [threading.Thread(target=work, args=(r,), name=f"pp-rank-{r}", daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    first = next((e for e in errors if e is not None and not (isinstance(e, RuntimeError) and "another pipeline rank failed" in str(e))),
                 None) or next((e for e in errors if e is not None), None)
    if first is not None:
        raise first
    states = [results[r][0] for r in range(n)]
    outs = []
    for k, o in enumerate(prog.outputs):
        if o[0] == "c":
            outs.append(o[1])
        else:
            merged = {}
            for r in range(n):
                merged.update(results[r][1][k])
            outs.append(merged)
    return states, outs
