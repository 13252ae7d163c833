"""Expert-parallel dispatch / combine as peer-memory kernels (Python side of ``csrc/moe_comm.cu``).

``dispatch`` = permutation into capacity slots + all-to-all in one pass (peer stores into the expert owner's
receive buffer); ``combine`` = all-to-all back + weighted gather-sum per token.  Both return ordinary tensors.
The reference has no mixture-of-experts support; this is part of what the B200 design adds.
"""
from __future__ import annotations

import ctypes
from typing import Any

import torch

from ..ops import native
from . import symm
from . import tp as tpmod


class JpbMoeDesc(ctypes.Structure):
    _fields_ = [("n_ranks", ctypes.c_int), ("rank", ctypes.c_int), ("epoch", ctypes.c_int), ("reserved_sms", ctypes.c_int),
                ("ctrl", ctypes.c_void_p * 8), ("recv", ctypes.c_void_p * 8)]


class _Workspace:
    CTRL = 1024

    def __init__(self, axis: str, nbytes: int):
        from ..mesh import MpmdMesh

        mesh = MpmdMesh.current()
        ranks = [d.process_index for d in mesh.peers_along(axis)]
        self.slot = (nbytes + 1023) // 1024 * 1024
        self.buf = symm.SymmetricBuffer(self.CTRL + 2 * self.slot, mesh.axis_group(axis), ranks)
        self.epoch = 0
        # with pipeline stages on other GPUs a few SMs stay out of the grid, so that point-to-point kernels of side
        # streams can start while these kernels wait for their peers (same rule as the fused GEMMs' workspaces)
        self.reserved_sms = symm.reserved_sms(mesh)

    def next_call(self) -> JpbMoeDesc:
        self.epoch += 1
        d = JpbMoeDesc()
        d.n_ranks, d.rank, d.epoch, d.reserved_sms = self.buf.n, self.buf.rank, self.epoch, self.reserved_sms
        for q in range(self.buf.n):
            d.ctrl[q] = self.buf.ptrs[q]
            d.recv[q] = self.buf.ptrs[q] + self.CTRL + (self.epoch & 1) * self.slot
        return d


_WS: dict[Any, _Workspace] = {}
_bound = False


def _lib():
    global _bound
    lib = native.load()
    if not _bound:
        p, i = ctypes.c_void_p, ctypes.c_int
        lib.jpb_moe_dispatch.argtypes = [p, p, p, p, i, i, i, i, ctypes.POINTER(JpbMoeDesc), p]
        lib.jpb_moe_combine.argtypes = [p, p, p, p, p, i, i, i, i, i, ctypes.POINTER(JpbMoeDesc), p]
        if lib.jpb_moe_desc_bytes() != ctypes.sizeof(JpbMoeDesc):
            raise native.NativeError("MoE call descriptor layout of the native library differs from the Python binding")
        _bound = True
    return lib


def _workspace(axis: str, nbytes: int) -> _Workspace:
    ws = _WS.get(axis)
    if ws is None or ws.slot < nbytes:
        if ws is not None:
            symm._RETIRED.append(ws)  # freed between steps, see symm.release_retired
        ws = _Workspace(axis, nbytes)
        _WS[axis] = ws
    return ws


def supported(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


def dispatch(x: torch.Tensor, src_of_slot: torch.Tensor, slot_scale, n_experts: int, capacity: int, axis: str) -> torch.Tensor:
    """x [T, d] bf16, src_of_slot [E*C] int32 (-1 = empty) -> [E_l, n*C, d] on every rank of ``axis``."""
    n = tpmod.axis_size(axis)
    d = x.shape[-1]
    x = x.contiguous()
    ws = _workspace(axis, n_experts * capacity * d * 2)
    desc = ws.next_call()
    out = torch.empty(n_experts // n, n * capacity, d, dtype=torch.bfloat16, device=x.device)
    rc = _lib().jpb_moe_dispatch(x.data_ptr(), src_of_slot.data_ptr(), None if slot_scale is None else slot_scale.data_ptr(),
                                 out.data_ptr(), x.shape[0], n_experts, capacity, d, ctypes.byref(desc), native._stream())
    native._check(rc, "jpb_moe_dispatch")
    return out


def combine(y: torch.Tensor, dest: torch.Tensor, weights, n_experts: int, capacity: int, top_k: int, axis: str,
            want_picked: bool):
    """y [E_l, n*C, d] bf16, dest [T*k] int32 (E*C = dropped), weights [T*k] fp32 or None -> (out [T, d], picked)"""
    d = y.shape[-1]
    T = dest.numel() // top_k
    y = y.contiguous()
    ws = _workspace(axis, n_experts * capacity * d * 2)
    desc = ws.next_call()
    out = torch.empty(T, d, dtype=torch.bfloat16, device=y.device)
    picked = torch.empty(T * top_k, d, dtype=torch.bfloat16, device=y.device) if want_picked else None
    rc = _lib().jpb_moe_combine(y.data_ptr(), dest.data_ptr(), None if weights is None else weights.data_ptr(), out.data_ptr(),
                                None if picked is None else picked.data_ptr(), T, top_k, n_experts, capacity, d,
                                ctypes.byref(desc), native._stream())
    native._check(rc, "jpb_moe_combine")
    return out, picked
