"""Fused tensor-parallel GEMMs: all-gather→GEMM and GEMM→reduce-scatter in one sm_100a kernel each.

Python side of ``csrc/gemm_comm_sm100.cu``: picks the symmetric workspace of the mesh axis, fills the call
descriptor (epoch, buffer parity, peer pointers) and launches; the kernel itself pushes this rank's shard to
the peers, so no staging copy runs around it.  Shapes the kernel does not cover (token counts that are not a multiple of
128 x ranks, feature counts that are not a multiple of 8) fall back to the NCCL twin in ``tp.py`` — loudly
countable through ``FALLBACKS``.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import core as ops
from ..ops import native
from . import symm
from . import tp as tpmod

FALLBACKS = [0]
_bound = False

GATHER_ROWS, GATHER_RED = 1, 2


def _lib():
    global _bound
    lib = native.load()
    if not _bound:
        p, i = ctypes.c_void_p, ctypes.c_int
        lib.jpb_comm_gemm.argtypes = [p, p, p, p] + [i] * 11 + [ctypes.POINTER(symm.JpbCommDesc), p, p]
        lib.jpb_memcpy_async.argtypes = [p, p, ctypes.c_longlong, p]
        _bound = True
    return lib


def _bf16_2d(t: torch.Tensor) -> torch.Tensor:
    t = t.reshape(-1, t.shape[-1])
    if t.dtype != torch.bfloat16:
        raise native.NativeError(f"fused tensor-parallel GEMMs take bfloat16, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _launch(a, b, out, bias, M, N, K, lda, ldb, a_mn, b_mn, accumulate, desc, gather_out=None):
    rc = _lib().jpb_comm_gemm(
        None if a is None else a.data_ptr(), None if b is None else b.data_ptr(), out.data_ptr(),
        None if bias is None else bias.data_ptr(), M, N, K, lda, ldb, out.stride(0), int(a_mn), int(b_mn),
        int(out.dtype == torch.float32), int(accumulate), int(bias is not None and bias.dtype == torch.float32),
        ctypes.byref(desc), None if gather_out is None else gather_out.data_ptr(), native._stream())
    native._check(rc, "jpb_comm_gemm")


def _rows_ok(rows_total: int, n: int) -> bool:
    return rows_total % (128 * n) == 0


def ag_linear(x, w, bias, axis):
    """y = all_gather_rows(x) @ w^T (+ bias)"""
    n = tpmod.axis_size(axis)
    x2, w2 = _bf16_2d(x), _bf16_2d(w)
    Ml, K = x2.shape
    M, N = Ml * n, w2.shape[0]
    if not _rows_ok(M, n) or K % 8 or N % 8:
        FALLBACKS[0] += 1
        return ops.linear(tpmod._all_gather_rows(x, axis), w, bias)
    ws = symm.workspace_for(axis, M * K * 2, 0)
    desc = ws.next_call(GATHER_ROWS, False, False)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    _launch(x2, w2, out, bias.contiguous() if bias is not None else None, M, N, K, K, w2.stride(0), False, False, False, desc)
    return out


def ag_dgrad(dy_shard, w, axis):
    """(dx, dy_full): dy_full = all_gather_rows(dy_shard), dx = dy_full @ w"""
    n = tpmod.axis_size(axis)
    dy2, w2 = _bf16_2d(dy_shard), _bf16_2d(w)  # w: [Nred, Kout]
    Ml, Nred = dy2.shape
    M, Kout = Ml * n, w2.shape[1]
    if not _rows_ok(M, n) or Nred % 8 or Kout % 8:
        FALLBACKS[0] += 1
        full = tpmod._all_gather_rows(dy_shard, axis)
        return ops.linear_dgrad(full, w), full
    ws = symm.workspace_for(axis, M * Nred * 2, 0)
    desc = ws.next_call(GATHER_ROWS, False, False)
    dx = torch.empty(M, Kout, dtype=torch.bfloat16, device=dy_shard.device)
    # the comm warps also assemble the gathered dy (the weight gradient needs it) while the tensor cores work
    full = torch.empty(M, Nred, dtype=torch.bfloat16, device=dy_shard.device)
    _launch(dy2, w2, dx, None, M, Kout, Nred, Nred, w2.stride(0), False, True, False, desc, gather_out=full)
    return dx, full


def ag_wgrad(dy, x_shard, axis, out_dtype=None, acc=None):
    """dW = dy^T @ all_gather_rows(x_shard); the gather runs along the reduction (token) dimension.  With ``acc``
    (fp32, same shape) the product is added into it by the kernel's accumulate epilogue and ``acc`` is returned."""
    n = tpmod.axis_size(axis)
    dy2, x2 = _bf16_2d(dy), _bf16_2d(x_shard)
    T, Nout = dy2.shape
    Tl, Kin = x2.shape
    out_dtype = out_dtype or torch.bfloat16
    if T != Tl * n or T % (64 * n) or Nout % 8 or Kin % 8 or (n * (Tl // 64)) > 4096:
        FALLBACKS[0] += 1
        return ops.linear_wgrad(dy, tpmod._all_gather_rows(x_shard, axis), out_dtype)
    ws = symm.workspace_for(axis, T * Kin * 2, 0)
    desc = ws.next_call(GATHER_RED, True, False)
    accumulate = acc is not None and acc.dtype == torch.float32 and out_dtype == torch.float32
    out = acc if accumulate else torch.empty(Nout, Kin, dtype=out_dtype, device=dy.device)
    _launch(dy2, x2, out, None, Nout, Kin, T, Nout, Kin, True, True, accumulate, desc)
    return out


def linear_rs(x, w, axis):
    """y_shard = reduce_scatter_rows(x @ w^T)"""
    n = tpmod.axis_size(axis)
    x2, w2 = _bf16_2d(x), _bf16_2d(w)
    M, K = x2.shape
    N = w2.shape[0]
    if not _rows_ok(M, n) or K % 8 or N % 8:
        FALLBACKS[0] += 1
        return tpmod._reduce_scatter_rows(ops.linear(x, w, None), axis)
    ws = symm.workspace_for(axis, 0, M * N * 2)
    desc = ws.next_call(0, False, True)
    out = torch.empty(M // n, N, dtype=torch.bfloat16, device=x.device)
    _launch(x2, w2, out, None, M, N, K, x2.stride(0), w2.stride(0), False, False, False, desc)
    return out


def dgrad_rs(dy, w, axis):
    """dx_shard = reduce_scatter_rows(dy @ w)"""
    n = tpmod.axis_size(axis)
    dy2, w2 = _bf16_2d(dy), _bf16_2d(w)  # w: [Nred, Kout]
    M, Nred = dy2.shape
    Kout = w2.shape[1]
    if not _rows_ok(M, n) or Nred % 8 or Kout % 8:
        FALLBACKS[0] += 1
        return tpmod._reduce_scatter_rows(ops.linear_dgrad(dy, w), axis)
    ws = symm.workspace_for(axis, 0, M * Kout * 2)
    desc = ws.next_call(0, False, True)
    out = torch.empty(M // n, Kout, dtype=torch.bfloat16, device=dy.device)
    _launch(dy2, w2, out, None, M, Kout, Nred, dy2.stride(0), w2.stride(0), False, True, False, desc)
    return out


# ---- all-reduce over peer memory (gradient sync) -----------------------------------------------------------------
class _AllReduceDesc(ctypes.Structure):
    _fields_ = [("n_ranks", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_int), ("dtype", ctypes.c_int),
                ("n", ctypes.c_longlong), ("scale", ctypes.c_float), ("counter_target", ctypes.c_uint),
                ("x", ctypes.c_void_p * 8), ("ctrl", ctypes.c_void_p * 8), ("out", ctypes.c_void_p), ("grid", ctypes.c_int),
                ("mode", ctypes.c_int)]


class _AllReduceWorkspace:
    CTRL = 1024

    def __init__(self, group, ranks: list, nbytes: int):
        self.slot = (nbytes + 1023) // 1024 * 1024
        self.buf = symm.SymmetricBuffer(self.CTRL + 2 * self.slot, group, ranks)
        self.epoch = 0
        self.ctas = 0


_AR_WS: dict = {}
AR_MIN_BYTES = 1 << 20  # smaller tensors are latency-bound: leave them to NCCL


def all_reduce(x: torch.Tensor, axis: str, scale: float = 1.0) -> torch.Tensor:
    """scale * sum over the ranks of mesh axis ``axis``; fp32 or bf16, any shape (padded internally)."""
    from ..mesh import MpmdMesh

    mesh = MpmdMesh.current()
    ranks = [d.process_index for d in mesh.peers_along(axis)]
    return all_reduce_group(x, mesh.axis_group(axis), ranks, scale)


def all_reduce_group(x: torch.Tensor, group, ranks: list, scale: float = 1.0) -> torch.Tensor:
    """scale * sum over the processes ``ranks`` (global ranks, same order everywhere) of process group ``group``:
    one kernel over NVLink peer memory (reduce-scatter + all-gather with direct peer loads).  Used for the
    gradient sync over a mesh axis and for cross-stage all-reduces (tied weights, global norms)."""
    flat = x.contiguous().view(-1)
    out = _peer_collective(flat, group, ranks, scale, 0)
    return out[:flat.numel()].view(x.shape)


def shard_numel(numel: int, n_ranks: int) -> int:
    """Elements per rank when a flat tensor of ``numel`` elements is split over ``n_ranks`` (padded so that every
    slice is a whole number of 16-byte vectors for 2- and 4-byte types alike)."""
    return (numel + 8 * n_ranks - 1) // (8 * n_ranks) * 8


def reduce_scatter_flat(x: torch.Tensor, axis: str, scale: float = 1.0) -> torch.Tensor:
    """This rank's slice ``[shard_numel]`` of scale * sum over the ranks of ``axis`` of the flattened ``x`` (zero
    padded): the first half of the one-kernel all-reduce, for gradients of parameters whose optimizer state is
    sharded over the axis."""
    from ..mesh import MpmdMesh

    mesh = MpmdMesh.current()
    ranks = [d.process_index for d in mesh.peers_along(axis)]
    return _peer_collective(x.contiguous().view(-1), mesh.axis_group(axis), ranks, scale, 1)


def all_gather_flat(shard: torch.Tensor, axis: str) -> torch.Tensor:
    """Concatenation ``[n_ranks * shard.numel()]`` of every rank's flat ``shard`` (equal sizes, a multiple of 8
    elements): the second half of the one-kernel all-reduce, for updated parameters gathered from the owners of
    their shards."""
    from ..mesh import MpmdMesh

    mesh = MpmdMesh.current()
    ranks = [d.process_index for d in mesh.peers_along(axis)]
    return _peer_collective(shard.contiguous().view(-1), mesh.axis_group(axis), ranks, 1.0, 2)


def _peer_collective(flat: torch.Tensor, group, ranks: list, scale: float, mode: int) -> torch.Tensor:
    """mode 0: all-reduce ``flat`` -> padded [n]; 1: reduce-scatter -> [n / n_ranks]; 2: all-gather of equal
    slices -> [n_ranks * flat.numel()]."""
    lib = _lib()
    lib.jpb_allreduce.argtypes = [ctypes.POINTER(_AllReduceDesc), ctypes.c_void_p]
    lib.jpb_allreduce_grid2.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_int]
    if lib.jpb_allreduce_desc_bytes() != ctypes.sizeof(_AllReduceDesc):
        raise native.NativeError("all-reduce call descriptor layout of the native library differs from the Python binding")
    n_ranks = len(ranks)
    if flat.dtype not in (torch.float32, torch.bfloat16):
        raise native.NativeError(f"peer-memory collectives take float32 or bfloat16, got {flat.dtype}")
    es = flat.element_size()
    vn = 16 // es
    if mode == 2:
        if flat.numel() % vn:
            raise native.NativeError("all_gather_flat needs slices of whole 16-byte vectors")
        n = flat.numel() * n_ranks
    else:
        quantum = (8 if mode == 1 else vn) * n_ranks
        n = (flat.numel() + quantum - 1) // quantum * quantum
    staged = flat.numel() if mode == 2 else n        # elements of X that this call uses
    nbytes = staged * es
    from ..runtime import executor as _ex
    from ..utils import config as _config

    side = _ex.OVERLAPPED[0]
    key = (tuple(ranks), "side") if side else tuple(ranks)
    ws = _AR_WS.get(key)
    if ws is None or ws.slot < nbytes:
        if ws is not None:
            symm._RETIRED.append(ws)  # freed between steps, see symm.release_retired
        ws = _AllReduceWorkspace(group, list(ranks), max(nbytes, 64 << 20))
        _AR_WS[key] = ws
    ws.epoch += 1
    parity = ws.epoch & 1
    d = _AllReduceDesc()
    d.n_ranks, d.rank, d.epoch, d.mode = ws.buf.n, ws.buf.rank, ws.epoch, mode
    d.dtype = 0 if flat.dtype == torch.float32 else 1
    d.n, d.scale = n, float(scale)
    d.grid = lib.jpb_allreduce_grid2(n, es, symm.reserved_sms())
    if side:   # runs beside the backward pass: a few CTAs are enough for a link and leave the SMs to the GEMMs
        d.grid = max(1, min(d.grid, int(_config.overlap_collective_ctas.value)))
    if mode == 0:
        ws.ctas += d.grid
    d.counter_target = ws.ctas & 0xFFFFFFFF
    for q in range(ws.buf.n):
        d.ctrl[q] = ws.buf.ptrs[q]
        d.x[q] = ws.buf.ptrs[q] + ws.CTRL + parity * ws.slot
    out = torch.empty(n // n_ranks if mode == 1 else n, dtype=flat.dtype, device=flat.device)
    d.out = out.data_ptr()
    stream = native._stream()
    mine = d.x[ws.buf.rank]
    native._check(lib.jpb_memcpy_async(mine, flat.data_ptr(), flat.numel() * es, stream), "stage", 0)
    if staged > flat.numel():
        lib.jpb_memset_async.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p]
        native._check(lib.jpb_memset_async(mine + flat.numel() * es, 0, (staged - flat.numel()) * es, stream), "pad", 0)
    native._check(lib.jpb_allreduce(ctypes.byref(d), stream), "jpb_allreduce")
    return out
