"""Symmetric (peer-mapped) GPU memory for the fused compute+collective kernels.

A :class:`SymmetricBuffer` is one ``cudaMalloc`` allocation of the same size on every rank of a process
group whose CUDA IPC handles have been exchanged, so that each process holds a device pointer to every
peer's copy (NVLink peer access).  A :class:`CommWorkspace` bundles what one family of fused GEMMs needs:
a control block of flags, a double-buffered gather buffer and a double-buffered receive buffer, plus the
host-side epoch / counter bookkeeping the kernels' flag protocol relies on.  Allocation and rendezvous
happen once per (group, shape) and are reused by every layer.

The reference has no counterpart (its collectives are XLA's); this is the layer the B200 design adds.
"""
from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from ..ops import native


class SymmetricBuffer:
    """``nbytes`` usable bytes on every rank of ``group``, each rank's copy mapped into every other rank's
    address space.  The allocation carries a guard band of ``GUARD`` bytes on either side of the usable range,
    filled with a pattern: ``check_canaries()`` reads them back, so a kernel that wrote outside its buffer (here
    or from a peer) is caught on the host without any tool that instruments the GPU."""

    GUARD = 256
    PATTERN = 0xA5
    LIVE: list = []   # every buffer of this process that has not been closed (what check_all_canaries walks)

    def __init__(self, nbytes: int, group, group_ranks: list[int]):
        lib = native.load()
        lib.jpb_ipc_alloc2.argtypes = [ctypes.c_longlong, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p, ctypes.c_void_p]
        lib.jpb_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
        lib.jpb_ipc_close.argtypes = [ctypes.c_void_p]
        lib.jpb_ipc_free.argtypes = [ctypes.c_void_p]
        lib.jpb_memset_async.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p]
        lib.jpb_memcpy_async.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
        self.lib = lib
        self.nbytes = nbytes
        self.group = group
        self.n = len(group_ranks)
        self.rank = group_ranks.index(dist.get_rank())
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        # zero-filled on the current stream, the stream of the guard fills below and of the caller's first use
        stream = native._stream()
        native._check(lib.jpb_ipc_alloc2(nbytes + 2 * self.GUARD, ctypes.byref(ptr), handle, stream), "jpb_ipc_alloc", 0)
        self.local_base = ptr.value
        native._check(lib.jpb_memset_async(self.local_base, self.PATTERN, self.GUARD, stream), "guard", 0)
        native._check(lib.jpb_memset_async(self.local_base + self.GUARD + nbytes, self.PATTERN, self.GUARD, stream), "guard", 0)
        handles: list[Any] = [None] * self.n
        dist.all_gather_object(handles, handle.raw, group=group)
        self.bases: list[int] = []
        for q, h in enumerate(handles):
            if q == self.rank:
                self.bases.append(self.local_base)
                continue
            peer = ctypes.c_void_p()
            native._check(lib.jpb_ipc_open(h, ctypes.byref(peer)), "jpb_ipc_open", 0)
            self.bases.append(peer.value)
        self.ptrs: list[int] = [b + self.GUARD for b in self.bases]   # usable range of every rank's copy
        self.local_ptr = self.ptrs[self.rank]
        # peers may write into this buffer as soon as they leave the barrier; only the current stream is
        # synchronised (a device-wide synchronisation would also wait for receives of a pipeline that are
        # posted ahead of time on side streams and cannot complete before this rank moves on)
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=group)
        SymmetricBuffer.LIVE.append(self)

    def _guards(self) -> torch.Tensor:
        host = torch.empty(2 * self.GUARD, dtype=torch.uint8, device="cuda")
        stream = native._stream()
        self.lib.jpb_memcpy_async(host.data_ptr(), self.local_base, self.GUARD, stream)
        self.lib.jpb_memcpy_async(host.data_ptr() + self.GUARD, self.local_base + self.GUARD + self.nbytes, self.GUARD, stream)
        return host.cpu()

    def check_canaries(self) -> bool:
        """True iff both guard bands of the local copy still hold the pattern (synchronises the current stream)."""
        return bool((self._guards() == self.PATTERN).all())

    def canary_report(self) -> str | None:
        """None if the guard bands are intact, else which band was overwritten, where and with what."""
        g = self._guards()
        bad = (g != self.PATTERN).nonzero().flatten().tolist()
        if not bad:
            return None
        side = lambda i: f"front band byte {i}" if i < self.GUARD else f"back band byte {i - self.GUARD}"
        vals = [int(g[i]) for i in bad[:8]]
        return (f"symmetric buffer of {self.nbytes} bytes ({self.n} ranks, rank {self.rank}): {len(bad)} guard bytes "
                f"overwritten, first at {side(bad[0])}, last at {side(bad[-1])}, values {vals}")

    def close(self):
        for q, b in enumerate(self.bases):
            if q != self.rank and b:
                self.lib.jpb_ipc_close(b)
        if self.local_base:
            self.lib.jpb_ipc_free(self.local_base)
        self.bases, self.ptrs, self.local_base, self.local_ptr = [], [], None, None
        if self in SymmetricBuffer.LIVE:
            SymmetricBuffer.LIVE.remove(self)


def check_all_canaries() -> bool:
    """Guard bands of every symmetric buffer of this process that is still allocated: the fused GEMM workspaces, the
    all-reduce / reduce-scatter / all-gather workspaces and the expert-parallel ones (every :class:`SymmetricBuffer`
    registers itself; closed and released buffers drop out)."""
    return all(buf.check_canaries() for buf in list(SymmetricBuffer.LIVE) if buf.local_base)


def canary_reports() -> list:
    """One line per symmetric buffer of this process whose guard bands were overwritten."""
    out = []
    for buf in list(SymmetricBuffer.LIVE):
        if buf.local_base:
            r = buf.canary_report()
            if r:
                out.append(r)
    return out


def reserved_sms(mesh=None) -> int:
    """SMs that kernels whose CTAs wait for peers leave free when pipeline stages live on other GPUs: point-to-point
    kernels of side streams must be able to start while such a kernel waits."""
    from ..mesh import MpmdMesh
    from ..utils import config

    if mesh is None:
        if not MpmdMesh.mesh_stack:
            return 0
        mesh = MpmdMesh.current()
    return int(config.comm_reserved_sms.value) if mesh.mpmd_dim > 1 else 0


class JpbCommDesc(ctypes.Structure):
    _fields_ = [
        ("n_ranks", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_int), ("gather", ctypes.c_int),
        ("gathered_is_b", ctypes.c_int), ("scatter", ctypes.c_int), ("max_ctas", ctypes.c_int),
        ("ctrl", ctypes.c_void_p * 8), ("g", ctypes.c_void_p * 8), ("r", ctypes.c_void_p * 8),
    ]


class CommWorkspace:
    """Control block + double-buffered gather (G) and receive (R) buffers for one process group."""

    def __init__(self, group, group_ranks: list[int], g_bytes: int, r_bytes: int):
        lib = native.load()
        lib.jpb_comm_ctrl_bytes.restype = ctypes.c_longlong
        if lib.jpb_comm_desc_bytes() != ctypes.sizeof(JpbCommDesc):
            raise native.NativeError("call descriptor layout of the native library differs from the Python binding")
        align = lambda x: (x + 1023) // 1024 * 1024
        self.ctrl_bytes = align(lib.jpb_comm_ctrl_bytes())
        self.g_bytes, self.r_bytes = align(max(g_bytes, 16)), align(max(r_bytes, 16))
        total = self.ctrl_bytes + 2 * self.g_bytes + 2 * self.r_bytes
        self.buf = SymmetricBuffer(total, group, group_ranks)
        self.n, self.rank = self.buf.n, self.buf.rank
        self.epoch = 0
        # With pipeline stages on other GPUs, point-to-point kernels on side streams must be able to start
        # while a fused kernel waits for its tensor-parallel peer: keep a few SMs out of the persistent grid.
        from ..mesh import MpmdMesh
        from ..utils import config

        mesh = MpmdMesh.current()
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        reserve = reserved_sms(mesh)
        self.max_ctas = max(1, sms - reserve) if reserve > 0 else 0

    def next_call(self, gather: int, gathered_is_b: bool, scatter: bool) -> JpbCommDesc:
        """Descriptor of the next fused call.  Every call both sends to and receives from every peer, and a
        rank's calls run in stream order; together that keeps a peer at most one call ahead, which is what the
        double buffering by call parity and the ever-growing epoch in the flags rely on."""
        self.epoch += 1
        parity = self.epoch & 1
        d = JpbCommDesc()
        d.n_ranks, d.rank, d.epoch = self.n, self.rank, self.epoch
        d.gather, d.gathered_is_b, d.scatter = gather, int(gathered_is_b), int(scatter)
        d.max_ctas = self.max_ctas
        for q in range(self.n):
            base = self.buf.ptrs[q]
            d.ctrl[q] = base
            d.g[q] = base + self.ctrl_bytes + parity * self.g_bytes
            d.r[q] = base + self.ctrl_bytes + 2 * self.g_bytes + parity * self.r_bytes
        return d


_WORKSPACES: dict[Any, CommWorkspace] = {}


def workspace_for(axis: str, g_bytes: int, r_bytes: int) -> CommWorkspace:
    """One workspace per mesh axis, grown (re-allocated collectively) when a larger shape shows up.  All
    ranks of the axis call this with the same arguments in the same order."""
    from ..mesh import MpmdMesh

    mesh = MpmdMesh.current()
    group = mesh.axis_group(axis)
    ranks = [d.process_index for d in mesh.peers_along(axis)]
    key = (axis, tuple(ranks))
    ws = _WORKSPACES.get(key)
    if ws is None or ws.g_bytes < g_bytes or ws.r_bytes < r_bytes:
        if ws is not None:
            # The outgrown workspace is retired, not freed: cudaFree and closing IPC mappings synchronise the
            # device, which must not happen while receives of a pipeline step are pending on side streams.
            g_bytes, r_bytes = max(g_bytes, ws.g_bytes), max(r_bytes, ws.r_bytes)
            _RETIRED.append(ws)
        ws = CommWorkspace(group, ranks, g_bytes, r_bytes)
        _WORKSPACES[key] = ws
    return ws


_RETIRED: list = []


def release_retired() -> None:
    """Free the workspaces that were outgrown.  Collective over every group that retired one: call it between
    steps with nothing in flight (outgrown buffers are small next to HBM, so never calling it is fine too)."""
    if not _RETIRED:
        return
    torch.cuda.synchronize()
    for ws in _RETIRED:
        dist.barrier(group=ws.buf.group)   # every importer is done with the mapping ...
        for q, base in enumerate(ws.buf.bases):
            if q != ws.buf.rank and base:
                ws.buf.lib.jpb_ipc_close(base)
        dist.barrier(group=ws.buf.group)   # ... and has closed it before the owner frees the memory
        ws.buf.lib.jpb_ipc_free(ws.buf.local_base)
        ws.buf.bases, ws.buf.ptrs, ws.buf.local_base, ws.buf.local_ptr = [], [], None, None
        if ws.buf in SymmetricBuffer.LIVE:
            SymmetricBuffer.LIVE.remove(ws.buf)
    _RETIRED.clear()
