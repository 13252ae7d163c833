"""Run-time configuration flags read from the environment.

Behavioural counterpart of the reference's flag classes (src/jaxpp/utils.py:35-113) and its
flag list (src/jaxpp/env_vars.py:3-22): a flag is parsed lazily from ``os.environ`` the first
time ``.value`` is read, the parsed value is remembered, and code can override it for a
dynamic extent with ``with flag.set(v):``.  Flag names keep the ``JAXPP_`` prefix so that
launch scripts written for the reference keep working.
"""
from __future__ import annotations

import contextlib
import math
import os
from typing import Generic, Iterator, TypeVar

T = TypeVar("T")
_UNSET = object()


class OverwriteableVar(Generic[T]):
    """A value holder with a default and a scoped override."""

    def __init__(self, default_value: T | None = None):
        self.default_value = default_value
        self._override = _UNSET

    def __bool__(self):
        # Guards against ``if flag:`` (always true for an object) instead of ``if flag.value:``.
        raise ValueError("Variable used as truthy value")

    @contextlib.contextmanager
    def set(self, to: T) -> Iterator[None]:
        saved = self._override
        self._override = to
        try:
            yield
        finally:
            self._override = saved

    @property
    def value(self) -> T:
        if self._override is not _UNSET:
            return self._override  # type: ignore[return-value]
        assert self.default_value is not None
        return self.default_value


class EnvVar(OverwriteableVar[T]):
    """Flag backed by an environment variable; the environment is consulted once."""

    def __init__(self, env_key: str, default_value: T | None = None, no_effect: str | None = None):
        super().__init__(default_value)
        self.env_key = env_key
        self._cached = _UNSET
        # flags kept only so that launch scripts and code written for the reference keep working: the reason why
        # the setting changes nothing here (``warn_about_flags_without_effect`` reports a non-default value)
        self.no_effect = no_effect

    def parse(self, text: str) -> T | None:  # pragma: no cover - overridden
        raise NotImplementedError

    @property
    def value(self) -> T:
        if self._override is not _UNSET:
            return self._override  # type: ignore[return-value]
        if self._cached is _UNSET:
            raw = os.getenv(self.env_key)
            if raw is None:
                assert self.default_value is not None
                self._cached = self.default_value
            else:
                parsed = self.parse(raw)
                if parsed is None:
                    raise ValueError(f"Unsupported value {self.env_key}={raw}")
                self._cached = parsed
        return self._cached  # type: ignore[return-value]


_TRUE = {"true", "1", "t", "y", "yes"}
_FALSE = {"false", "0", "f", "n", "no"}


def parse_bool(s: str) -> bool | None:
    low = s.lower()
    if low in _TRUE:
        return True
    if low in _FALSE:
        return False
    return None


class BoolEnvVar(EnvVar[bool]):
    def parse(self, text: str) -> bool | None:
        return parse_bool(text)


class StrEnvVar(EnvVar[str]):
    def parse(self, text: str) -> str | None:
        return text


class IntEnvVar(EnvVar[int]):
    def parse(self, text: str) -> int | None:
        try:
            return int(text)
        except ValueError:
            return None


# --- flags (same names and defaults as the reference, env_vars.py:3-22) -----------------
share_donation = BoolEnvVar(
    "JAXPP_SHARE_DONATION", True,
    no_effect="donation is a per-call list handed to the interpreter, not part of an executable: tasks that share code "
              "never recompile because their donation differs")
enable_local_propagation = BoolEnvVar(
    "JAXPP_ENABLE_LOCAL_PROPAGATION", False,
    no_effect="shardings are explicit (tensor-/data-/expert-parallel layers state them); nothing is inferred per task")
enable_licm = BoolEnvVar("JAXPP_ENABLE_LICM", False)
dump_dir = StrEnvVar("JAXPP_DUMP_DIR", "")
# inf (the default) = sent buffers are only collected at the end of the step.
transfer_done_delay = IntEnvVar("JAXPP_TRANSFER_DONE_DELAY", math.inf)  # type: ignore[arg-type]
disable_schedule_task_fusion = BoolEnvVar("JAXPP_DISABLE_SCHEDULE_TASK_FUSION", False)
# Common-subexpression elimination (JAXPP_ENABLE_LICM) never replaces an op of the backward pass by one of the forward pass,
# which is what keeps a recomputed block recomputed; this flag lifts the barrier.
disable_prevent_cse = BoolEnvVar("JAXPP_DISABLE_PREVENT_CSE", False)
directional_communicators = BoolEnvVar(
    "JAXPP_DIRECTIONAL_COMMUNICATORS", False,
    no_effect="point-to-point transfers always use one communicator per direction of a pair of pipeline ranks: "
              "receives are posted ahead of time here, and on a shared communicator one would hold back the sends "
              "issued after it")
conservative_loop_clustering = BoolEnvVar("JAXPP_CONSERVATIVE_LOOP_CLUSTERING", True)
debug_skip_propagation = BoolEnvVar(
    "JAXPP_DEBUG_SKIP_PROPAGATION", False, no_effect="there is no sharding propagation to skip (shardings are explicit)")
# run the per-rank programs of the multi-process path as threads of one process (runtime/local_comm.py)
debug_force_mpmdify = BoolEnvVar("JAXPP_DEBUG_FORCE_MPMDIFY", False)
fast_infer_shardings = BoolEnvVar(
    "JAXPP_FAST_INFER_SHARDINGS", False, no_effect="there is no throw-away driver compile that infers shardings")
enable_check_ir = BoolEnvVar("JAXPP_ENABLE_CHECK_JAXPR", False)

# --- flags that only exist in this framework ----------------------------------------------
# Use the hand-written sm_100a kernels (1) or the ATen reference implementations (0) on CUDA.
use_native_kernels = BoolEnvVar("JAXPP_B200_NATIVE", True)
# Use fused compute+collective kernels over peer memory (1) or the NCCL-only twins (0).
use_fused_collectives = BoolEnvVar("JAXPP_B200_FUSED_COLLECTIVES", True)
# SMs the fused compute+collective kernels leave free when pipeline stages run on other GPUs, so that the
# point-to-point kernels of side streams can start while a fused kernel waits for its tensor-parallel peer.
comm_reserved_sms = IntEnvVar("JAXPP_B200_COMM_RESERVED_SMS", 4)
# Point-to-point backend of the multi-controller runtime on GPUs: "torch" (torch.distributed batch_isend_irecv) or
# "native" (2-rank NCCL communicators driven through the C ABI of the native library).
p2p_backend = StrEnvVar("JAXPP_B200_P2P", "torch")
# Rewrite "norm backward, then add the residual-path gradient" into one kernel (compiler/peephole.py).
fuse_norm_backward_adds = BoolEnvVar("JAXPP_B200_FUSE_NORM_BWD_ADD", True)
# Let weight-gradient GEMMs add straight into the microbatch loop's accumulators (ops/sink.py).
wgrad_sinks = BoolEnvVar("JAXPP_B200_WGRAD_SINKS", True)
# Hoisting with scarce memory: cheap ops that only expand their operands go back into the loop (needs JAXPP_ENABLE_LICM).
licm_memory_scarce = BoolEnvVar("JAXPP_B200_LICM_MEMORY_SCARCE", True)
# Zero-bubble split: move left-over cheap, non-expanding, non-GEMM ops into the activation-gradient half.
zb_memory_scarce = BoolEnvVar("JAXPP_B200_ZB_MEMORY_SCARCE", True)
# Zero-bubble split: bytes of operands that deferred weight-gradient GEMMs may keep alive per (stage, microbatch);
# weight gradients beyond the budget run with the activation gradients.  Negative = no limit.
zb_defer_bytes = IntEnvVar("JAXPP_B200_ZB_DEFER_BYTES", -1)
# Issue the data-parallel gradient collectives (all-reduce, or reduce-scatter with sharded optimizer state) from inside
# the backward task that adds the last microbatch's weight gradient, on a side stream, instead of after the loop.
overlap_grad_reduce = BoolEnvVar("JAXPP_B200_OVERLAP_GRAD_REDUCE", True)
# CTAs of a peer-memory collective that runs beside compute kernels (it shares the SMs with them).
overlap_collective_ctas = IntEnvVar("JAXPP_B200_OVERLAP_CTAS", 32)
# Expert GEMMs of a mixture-of-experts layer skip what is made only of unused capacity slots.  0: nothing; 1: the 64-row
# reduction blocks of the weight gradient (measured 17 % faster at 80 % fill); 2: also output tiles of the forward and
# input-gradient GEMMs (faster only when empty tiles come in runs that keep the CTAs' walk over the tiles in step:
# 1.7x at 50 % fill, nothing at 80 % fill in one block per expert).
moe_skip_empty_slots = IntEnvVar("JAXPP_B200_MOE_SKIP_EMPTY_SLOTS", 1)
# Seconds a rank may go without a heartbeat before the watchdog reports it.
heartbeat_timeout_s = IntEnvVar("JAXPP_B200_HEARTBEAT_TIMEOUT", 30)
# Wrap every task in an NVTX range named like the task (fwd_3__5, …) for timeline profilers.
nvtx_ranges = BoolEnvVar("JAXPP_B200_NVTX", False)


_WARNED: set = set()


def warn_about_flags_without_effect(log) -> None:
    """Tell the user once about every reference flag that is set to a non-default value but changes nothing here."""
    for name, var in list(globals().items()):
        if isinstance(var, EnvVar) and var.no_effect and name not in _WARNED:
            try:
                changed = var.value != var.default_value
            except ValueError:
                changed = True
            if changed:
                _WARNED.add(name)
                log.warning("%s is set but has no effect in this framework: %s", var.env_key, var.no_effect)
