"""Small helpers: timers, byte formatting, list utilities.

Covers the reference's general-purpose utilities (src/jaxpp/utils.py:115-383) that make
sense without JAX: ``log_elapsed_time``, ``hbytes``, ``groupby``, ``partition``,
``unzip_multi`` and the PartitionSpec helpers ``filter_axes`` / ``rm_size1_axes``.
"""
from __future__ import annotations

import contextlib
import logging
import time
from collections import defaultdict
from typing import Callable, Hashable, Iterable, Sequence, TypeVar

logger = logging.getLogger("jaxpp_b200")

A = TypeVar("A")
K = TypeVar("K", bound=Hashable)

_UNITS = ("B", "KiB", "MiB", "GiB", "TiB", "PiB")


def format_bytes(n: float) -> str:
    """Human readable size with binary units, two decimals above bytes."""
    n = float(n)
    sign = "-" if n < 0 else ""
    n = abs(n)
    unit = 0
    while n >= 1024.0 and unit < len(_UNITS) - 1:
        n /= 1024.0
        unit += 1
    if unit == 0:
        return f"{sign}{int(n)}{_UNITS[0]}"
    return f"{sign}{n:.2f}{_UNITS[unit]}"


def hbytes(sizes) -> str:
    """Format one byte count or an iterable of them (summed)."""
    if isinstance(sizes, (int, float)):
        return format_bytes(sizes)
    return format_bytes(sum(sizes))


@contextlib.contextmanager
def log_elapsed_time(event: str, msg: str | None = None, unit: str = "s", log: logging.Logger | None = None):
    """Log how long the ``with`` body took, tagged by ``event``.

    ``unit`` is ``"s"`` or ``"ms"``; anything else raises ``ValueError`` before the body runs.
    """
    if unit not in ("s", "ms"):
        raise ValueError(f"Unknown unit `{unit}`")
    log = log or logger
    t0 = time.perf_counter()
    try:
        yield
    finally:
        dt = time.perf_counter() - t0
        if unit == "ms":
            dt *= 1e3
        extra = f" {msg}" if msg else ""
        log.info("[%s]%s took %.3f%s", event, extra, dt, unit)


def unzip_multi(xs: Sequence[Sequence], arity: int = 2) -> list[list]:
    """Transpose a list of ``arity``-tuples into ``arity`` lists (empty input → empty lists)."""
    if len(xs) == 0:
        return [[] for _ in range(arity)]
    if any(len(x) != arity for x in xs):
        raise AssertionError(f"every element must have length {arity}")
    return [list(col) for col in zip(*xs)]


def groupby(pairs: Iterable[tuple[K, A]]) -> dict[K, list[A]]:
    """Group ``(key, value)`` pairs by key, preserving first-seen key order."""
    out: dict[K, list[A]] = defaultdict(list)
    for k, v in pairs:
        out[k].append(v)
    return dict(out)


def partition(pred: Callable[[A], bool], xs: Iterable[A]) -> tuple[list[A], list[A]]:
    """Split into (elements satisfying ``pred``, the others), both in input order."""
    yes: list[A] = []
    no: list[A] = []
    for x in xs:
        (yes if pred(x) else no).append(x)
    return yes, no


def unique_in_order(xs: Iterable[A]) -> list[A]:
    seen = set()
    out = []
    for x in xs:
        if x not in seen:
            seen.add(x)
            out.append(x)
    return out


def _device_memory_lines() -> list[str]:
    import torch

    lines = []
    if not torch.cuda.is_available():
        return lines
    for i in range(torch.cuda.device_count()):
        free, limit = torch.cuda.mem_get_info(i)
        stats = torch.cuda.memory_stats(i)
        used = (limit - free) / 2 ** 30
        peak = stats.get("allocated_bytes.all.peak", 0) / 2 ** 30
        lines.append(f"\tUsing (GiB) {used:.2f} / {limit / 2 ** 30:.2f} ({used / (limit / 2 ** 30):.1%}) "
                     f"(peak allocated {peak:.2f} GiB) on cuda:{i}")
    return lines


@contextlib.contextmanager
def print_memstats(label: str, enabled: bool = False):
    """Print the device memory in use, its limit and the allocator's peak for every visible GPU before and after the
    ``with`` body (reference: utils.py:241-268).  Off unless ``enabled``; prints only the labels without a GPU."""
    if not enabled:
        yield
        return
    print(f"\nBefore: {label}:")
    for line in _device_memory_lines():
        print(line, flush=True)
    yield
    print(f"\nAfter: {label}:")
    for line in _device_memory_lines():
        print(line, flush=True)


def updated_named_sharding_mesh(shardings, new_mesh):
    """The same partition specs over ``new_mesh``: ``None`` entries pass through (reference: utils.py:223-238)."""
    from ..mesh import NamedSharding

    out = []
    for s in shardings:
        if s is None:
            out.append(None)
            continue
        if not isinstance(s, NamedSharding):
            raise TypeError(f"expected a NamedSharding or None, got {type(s).__name__}")
        out.append(NamedSharding(new_mesh, s.spec))
    return out
