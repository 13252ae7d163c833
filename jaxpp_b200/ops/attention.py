"""Bindings for the flash-attention kernels (tensors are [batch, seq, heads, head_dim], bf16)."""
from __future__ import annotations

import ctypes

import torch

from . import native

_c_int, _c_f, _c_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_bound = False


def _lib():
    global _bound
    lib = native.load()
    if not _bound:
        lib.jpb_attention_fwd.argtypes = [_c_p] * 5 + [_c_int] * 7 + [_c_f, _c_p]
        lib.jpb_attention_bwd.argtypes = [_c_p] * 11 + [_c_int] * 7 + [_c_f, _c_p]
        lib.jpb_attention_bwd_scratch_bytes.argtypes = [_c_int] * 6
        lib.jpb_attention_bwd_scratch_bytes.restype = ctypes.c_longlong
        _bound = True
    return lib


def _check_inputs(q, k, v):
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise native.NativeError(f"flash attention takes bfloat16 tensors, got {q.dtype}/{k.dtype}/{v.dtype}")
    if q.shape[-1] not in (64, 128):
        raise native.NativeError(f"head_dim must be 64 or 128, got {q.shape[-1]}")


def attention_fwd(q, k, v, causal: bool, scale: float):
    _check_inputs(q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    o = torch.empty_like(q)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device)
    rc = _lib().jpb_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, Sq, Sk, H, Hkv, D,
                                  int(causal), float(scale), native._stream())
    native._check(rc, "jpb_attention_fwd")
    return o, lse


def attention_bwd(do, q, k, v, o, lse, causal: bool, scale: float):
    _check_inputs(q, k, v)
    do, q, k, v, o, lse = (t.contiguous() for t in (do, q, k, v, o, lse))
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    lib = _lib()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    scratch = torch.empty(lib.jpb_attention_bwd_scratch_bytes(B, Sq, Sk, H, Hkv, D), dtype=torch.uint8, device=q.device)
    rc = lib.jpb_attention_bwd(do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                               dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), scratch.data_ptr(), None, B, Sq, Sk, H, Hkv, D,
                               int(causal), float(scale), native._stream())
    native._check(rc, "jpb_attention_bwd", 3)
    return dq, dk, dv
