"""Per-step metrics as JSON lines (the reference only logs through ``logging`` and prints by hand,
examples/tutorial.ipynb:173-198).

``StepMetrics`` times steps on the device (CUDA events on the launching stream; max over ranks when a process
group is up), derives tokens/s and the pipeline bubble from the per-task events the executor records, and
appends one JSON object per step to a file: step, loss, step_ms, tokens_per_s, bubble_pct, busy_ms, bytes sent
between stages, peak device memory.
"""
from __future__ import annotations

import json
import time
from typing import Any

import torch


class StepMetrics:
    def __init__(self, path: str | None, tokens_per_step: int, compiled=None, rank: int = 0):
        self.path, self.tokens_per_step, self.compiled, self.rank = path, tokens_per_step, compiled, rank
        self._fh = open(path, "a") if path and rank == 0 else None
        self._cuda = torch.cuda.is_available()
        self._t0 = None
        self._e0 = self._e1 = None
        self.history: list[dict] = []

    def begin(self):
        if self._cuda:
            self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._e0.record()
        self._t0 = time.perf_counter()

    def end(self, step: int, loss: float | None = None, **extra: Any) -> dict:
        if self._cuda:
            self._e1.record()
            self._e1.synchronize()
            ms = self._e0.elapsed_time(self._e1)
        else:
            ms = (time.perf_counter() - self._t0) * 1e3
        busy = None
        if self.compiled is not None and self.compiled.last_states:
            st = self.compiled.last_states
            if any(s.events for s in st):
                busy = max(s.busy_ms() for s in st)
        rec = {"step": step, "loss": loss, "step_ms": ms}
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([ms, busy if busy is not None else -1.0], dtype=torch.float64,
                             device="cuda" if dist.get_backend() == "nccl" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            rec["step_ms"], busy = float(t[0]), (float(t[1]) if float(t[1]) >= 0 else None)
        rec["tokens_per_s"] = self.tokens_per_step / (rec["step_ms"] / 1e3)
        if busy is not None:
            rec["busy_ms"] = busy
            rec["bubble_pct"] = max(0.0, 100.0 * (1.0 - busy / rec["step_ms"]))
        if self.compiled is not None:
            rec["transfer_bytes"] = self.compiled.program.stats()["transfer_bytes"]
        if self._cuda:
            rec["peak_mem_bytes"] = torch.cuda.max_memory_allocated()
        rec.update(extra)
        self.history.append(rec)
        if self._fh is not None:
            self._fh.write(json.dumps(rec) + "\n")
            self._fh.flush()
        return rec

    def close(self):
        if self._fh is not None:
            self._fh.close()
