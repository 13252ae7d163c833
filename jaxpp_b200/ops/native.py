"""ctypes bindings for the native sm_100a library (``jaxpp_b200/_native/libjaxpp_b200.so``).

Every function here takes and returns ``torch`` CUDA tensors, allocates outputs through torch's
caching allocator and launches on the *current* CUDA stream.  ``load()`` raises if the library is
missing: on a GPU machine the ops never silently fall back to a library or eager implementation.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_LIB: ctypes.CDLL | None = None
_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "_native", "libjaxpp_b200.so")

_c_int, _c_ll, _c_f, _c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def load() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    from ..csrc import build as _build

    if not _build.is_current():
        # a binary that does not match its sources has a different ABI than the bindings below: never load it
        import shutil

        if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
            _build.ensure_current()
        else:
            raise RuntimeError(
                f"native kernel library at {LIB_PATH} is missing or older than its sources and nvcc is not available; "
                "build it with `python -m jaxpp_b200.csrc.build` (or __graft_entry__.build())"
            )
    lib = ctypes.CDLL(LIB_PATH)
    lib.jpb_gemm_bf16.argtypes = [_c_p, _c_p, _c_p, _c_p] + [_c_int] * 11 + [_c_p]
    lib.jpb_norm_fwd.argtypes = [_c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_f, _c_p]
    lib.jpb_norm_bwd.argtypes = [_c_int, _c_int] + [_c_p] * 9 + [_c_int, _c_int, _c_p]
    lib.jpb_norm_bwd_scratch_elems.argtypes = [_c_int, _c_int]
    lib.jpb_norm_bwd_scratch_elems.restype = _c_ll
    lib.jpb_colsum_scratch_elems.argtypes = [_c_int, _c_int]
    lib.jpb_colsum_scratch_elems.restype = _c_ll
    lib.jpb_colsum.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p]
    lib.jpb_gelu.argtypes = [_c_int, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_p]
    lib.jpb_swiglu.argtypes = [_c_int, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_p]
    lib.jpb_rope.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p]
    lib.jpb_embedding_fwd.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p]
    lib.jpb_embedding_bwd.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p]
    lib.jpb_ce_fwd.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p]
    lib.jpb_ce_bwd.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p]
    lib.jpb_adamw.argtypes = [_c_int, _c_int] + [_c_p] * 9 + [_c_ll] + [_c_f] * 6 + [_c_p]
    lib.jpb_read_status.argtypes = [_c_int]
    lib.jpb_build_info.restype = ctypes.c_char_p
    for name in ("jpb_attention_fwd", "jpb_attention_bwd"):
        if hasattr(lib, name):
            getattr(lib, name).restype = _c_int
    _LIB = lib
    return lib


def is_available() -> bool:
    return os.path.exists(LIB_PATH)


class NativeError(RuntimeError):
    pass


# number of kernels of this library launched so far (benchmarks reset and read it)
LAUNCHES = [0]


def _check(rc: int, what: str, launches: int = 1):
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")
    LAUNCHES[0] += launches


def read_status(clear: bool = True) -> int:
    """Status word of the current device: non-zero after a kernel gave up on a bounded wait (1), rejected an
    argument (2) or timed out waiting for a peer GPU (3).  Synchronise the stream first."""
    return load().jpb_read_status(1 if clear else 0)


STATUS_NAMES = {1: "a bounded wait on an mbarrier ran out (JPB_ERR_WAIT_TIMEOUT)",
                2: "a kernel rejected an argument or met an out-of-range index (JPB_ERR_BAD_ARGUMENT)",
                3: "a bounded wait on a peer GPU's flag ran out (JPB_ERR_PEER_TIMEOUT)"}


class KernelStatusError(NativeError):
    """A kernel of the step reported through the device's status word that it gave up: its outputs are not valid."""

    def __init__(self, code: int, where: str = ""):
        self.code = code
        super().__init__(f"kernel status {code}{' after ' + where if where else ''}: "
                         f"{STATUS_NAMES.get(code, 'unknown status')}; the results of this step must not be used")


def raise_on_status(where: str = "", synchronize: bool = True) -> None:
    """Synchronise the current device and raise :class:`KernelStatusError` if any kernel of this library gave up
    since the last check.  A kernel that runs out of its wait budget returns early and leaves its outputs
    unwritten, so a training loop calls this once per step before it trusts (or checkpoints) the new state."""
    if synchronize and torch.cuda.is_available():
        torch.cuda.synchronize()
    code = read_status(clear=True)
    if code != 0:
        raise KernelStatusError(code, where)


def set_wait_budget_ms(ms: float) -> None:
    """Longest time a device-side wait of this library spins on the current device before its kernel gives up
    (default 4000 ms).  Applies to kernels launched afterwards."""
    lib = load()
    lib.jpb_set_wait_budget_ns.argtypes = [ctypes.c_ulonglong]
    rc = lib.jpb_set_wait_budget_ns(int(ms * 1e6))
    if rc != 0:
        raise NativeError(f"jpb_set_wait_budget_ns failed with code {rc}")


def _stream() -> int:
    """Raw handle of the current stream of the current device (the C getters: a ``torch.cuda.Stream`` object per launch
    costs more than the rest of a small op's wrapper)."""
    try:
        return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())
    except AttributeError:  # pragma: no cover - a torch build without the private getters
        return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise NativeError(f"native kernels support float32 and bfloat16, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _rows(t: torch.Tensor) -> int:
    return t.numel() // t.shape[-1]


# ---- GEMM ---------------------------------------------------------------------------------------------
def _as_2d_bf16(t: torch.Tensor) -> torch.Tensor:
    # the common case first (a contiguous bfloat16 matrix whose rows start on 16-byte boundaries): this function runs
    # two or three times per GEMM, and in launch-bound configurations the Python in front of a kernel is the step time
    if (t.dim() == 2 and t.dtype == torch.bfloat16 and t.is_contiguous() and not (t.shape[1] & 7)
            and not (t.data_ptr() & 15)):
        return t
    t2 = t.reshape(-1, t.shape[-1])
    if t2.dtype != torch.bfloat16:
        raise NativeError(f"the tcgen05 GEMM takes bfloat16 operands, got {t2.dtype}")
    if t2.shape[-1] % 8:
        # TMA wants rows that start on 16-byte boundaries: give a narrow operand (a router's [tokens, n_experts]
        # logits gradient, say) a row pitch that is a multiple of 8 elements; the extra columns are never addressed
        width = t2.shape[-1]
        padded = torch.zeros(t2.shape[0], (width + 7) // 8 * 8, dtype=t2.dtype, device=t2.device)
        padded[:, :width].copy_(t2)
        return padded[:, :width]
    if t2.stride(-1) != 1 or (t2.stride(0) % 8) or (t2.data_ptr() % 16):
        t2 = t2.contiguous()
    return t2


def gemm(a: torch.Tensor, b: torch.Tensor, M: int, N: int, K: int, a_mn: bool, b_mn: bool, out: torch.Tensor,
         bias: Optional[torch.Tensor] = None, accumulate: bool = False):
    """``out[M,N] (+)= A * B^T``.  ``a`` is [M,K] (or [K,M] when ``a_mn``), ``b`` is [N,K] (or [K,N] when ``b_mn``)."""
    lib = load()
    rc = lib.jpb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), _p(bias), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate),
        int(bias is not None and bias.dtype == torch.float32), _stream(),
    )
    _check(rc, "jpb_gemm_bf16")
    return out


def linear(x, w, bias):
    x2 = _as_2d_bf16(x)
    w2 = _as_2d_bf16(w)
    M, K = x2.shape
    N = w2.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    gemm(x2, w2, M, N, K, False, False, out, bias.contiguous() if bias is not None else None)
    return out if x.dim() == 2 else out.view(*x.shape[:-1], N)


def _counts_ok(counts, E) -> bool:
    return (counts is not None and counts.dtype == torch.int32 and counts.dim() == 2 and counts.shape[0] == E
            and counts.is_contiguous())


def _skip_rows() -> bool:
    """Row counts are used by the forward / input-gradient grouped GEMMs only on request (see the flag's comment)."""
    from ..utils import config

    return config.moe_skip_empty_slots.value >= 2


def _gemm_batched(a, b, out, batch, M, N, K, a_mn, b_mn, counts=None, seg_rows=0, count_k=False, accumulate=False):
    lib = load()
    if counts is not None:
        lib.jpb_gemm_bf16_grouped.argtypes = [_c_p, _c_p, _c_p] + [_c_int] * 11 + [_c_p] + [_c_int] * 3 + [_c_p]
        rc = lib.jpb_gemm_bf16_grouped(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, M, N, K, a.stride(-2), b.stride(-2),
                                       out.stride(-2), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate),
                                       counts.data_ptr(), seg_rows, counts.shape[1], int(count_k), _stream())
        _check(rc, "jpb_gemm_bf16_grouped")
        return out
    lib.jpb_gemm_bf16_batched.argtypes = [_c_p, _c_p, _c_p] + [_c_int] * 11 + [_c_p]
    rc = lib.jpb_gemm_bf16_batched(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, M, N, K, a.stride(-2), b.stride(-2),
                                   out.stride(-2), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), _stream())
    _check(rc, "jpb_gemm_bf16_batched")
    return out


def _batched_ok(*ts) -> bool:
    return all(t.dtype == torch.bfloat16 and t.dim() == 3 for t in ts)


def linear_batched(x, w, counts=None, seg_rows=0):
    """x [E, M, K], w [E, N, K] -> [E, M, N]; one grouped launch when the reduction length allows it.  ``counts``
    ([E, M / seg_rows] int32): rows of data at the start of each ``seg_rows``-row segment of a group; the rest of
    ``x`` is zero and the kernel neither loads nor multiplies tiles made of such rows only."""
    E, M, K = x.shape
    N = w.shape[1]
    if not _batched_ok(x, w) or K % 64 or K % 8:
        return torch.stack([linear(x[e], w[e], None) for e in range(E)], 0)
    x, w = x.contiguous(), w.contiguous()
    out = torch.empty(E, M, N, dtype=torch.bfloat16, device=x.device)
    if _counts_ok(counts, E) and seg_rows * counts.shape[1] == M and _skip_rows():
        return _gemm_batched(x, w, out, E, M, N, K, False, False, counts, seg_rows, False)
    return _gemm_batched(x, w, out, E, M, N, K, False, False)


def linear_dgrad_batched(dy, w, counts=None, seg_rows=0):
    """dy [E, M, N], w [E, N, K] -> [E, M, K] (reduction over N); ``counts`` as in :func:`linear_batched`."""
    E, M, N = dy.shape
    K = w.shape[2]
    if not _batched_ok(dy, w) or N % 64 or K % 8:
        return torch.stack([linear_dgrad(dy[e], w[e]) for e in range(E)], 0)
    dy, w = dy.contiguous(), w.contiguous()
    out = torch.empty(E, M, K, dtype=torch.bfloat16, device=dy.device)
    if _counts_ok(counts, E) and seg_rows * counts.shape[1] == M and _skip_rows():
        return _gemm_batched(dy, w, out, E, M, K, N, False, True, counts, seg_rows, False)
    return _gemm_batched(dy, w, out, E, M, K, N, False, True)


def linear_wgrad_batched(dy, x, out_dtype=None, counts=None, seg_rows=0, out=None, accumulate=False):
    """dy [E, M, N], x [E, M, K] -> [E, N, K] (reduction over the M tokens of each group).  With ``counts`` the
    reduction skips 64-row blocks that hold no data.  ``out`` (fp32, contiguous) with ``accumulate``: the product is
    added onto it in the GEMM's epilogue; None is returned when the shapes do not allow the grouped kernel."""
    E, M, N = dy.shape
    K = x.shape[2]
    if out is not None:
        if not _batched_ok(dy, x) or M % 64 or N % 8 or K % 8 or out.dtype != torch.float32 or not out.is_contiguous():
            return None
        dy, x = dy.contiguous(), x.contiguous()
        use_counts = _counts_ok(counts, E) and seg_rows * counts.shape[1] == M
        return _gemm_batched(dy, x, out, E, N, K, M, True, True, counts if use_counts else None, seg_rows, use_counts, accumulate)
    out_dtype = out_dtype or dy.dtype
    if not _batched_ok(dy, x) or M % 64 or N % 8 or K % 8 or out_dtype not in (torch.bfloat16, torch.float32):
        out = torch.empty(E, N, K, dtype=out_dtype, device=dy.device)
        for e in range(E):
            if out_dtype in (torch.bfloat16, torch.float32):
                linear_wgrad(dy[e], x[e], out=out[e])
            else:
                out[e] = linear_wgrad(dy[e], x[e]).to(out_dtype)
        return out
    dy, x = dy.contiguous(), x.contiguous()
    out = torch.empty(E, N, K, dtype=out_dtype, device=dy.device)
    if _counts_ok(counts, E) and seg_rows * counts.shape[1] == M:
        return _gemm_batched(dy, x, out, E, N, K, M, True, True, counts, seg_rows, True)
    return _gemm_batched(dy, x, out, E, N, K, M, True, True)


def linear_dgrad(dy, w):
    dy2 = _as_2d_bf16(dy)
    w2 = _as_2d_bf16(w)  # [N_out, K_in]: reduction over N_out, so w is the MN-major B operand
    M, Nred = dy2.shape
    Kout = w2.shape[1]
    out = torch.empty(M, Kout, dtype=torch.bfloat16, device=dy.device)
    gemm(dy2, w2, M, Kout, Nred, False, True, out)
    return out if dy.dim() == 2 else out.view(*dy.shape[:-1], Kout)


def linear_wgrad(dy, x, out: Optional[torch.Tensor] = None, accumulate: bool = False):
    dy2 = _as_2d_bf16(dy)
    x2 = _as_2d_bf16(x)
    tokens, Nout = dy2.shape
    Kin = x2.shape[1]
    if out is None:
        out = torch.empty(Nout, Kin, dtype=torch.bfloat16, device=dy.device)
    gemm(dy2, x2, Nout, Kin, tokens, True, True, out, accumulate=accumulate)
    return out


# ---- norms ----------------------------------------------------------------------------------------------
def rmsnorm(x, w, eps):
    x = x.contiguous()
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    _check(load().jpb_norm_fwd(0, _dt(x), x.data_ptr(), w.contiguous().data_ptr(), None, y.data_ptr(), None,
                               rstd.data_ptr(), _rows(x), x.shape[-1], float(eps), _stream()), "rmsnorm")
    return y, rstd


def norm_bwd_scratch(rows: int, H: int, device) -> torch.Tensor:
    n = load().jpb_norm_bwd_scratch_elems(rows, H)
    return torch.empty(n, dtype=torch.float32, device=device)


def rmsnorm_bwd(dy, x, w, rstd):
    dy, x, w = dy.contiguous(), x.contiguous(), w.contiguous()
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    rows, H = _rows(x), x.shape[-1]
    scratch = norm_bwd_scratch(rows, H, x.device)
    _check(load().jpb_norm_bwd(0, _dt(x), dy.data_ptr(), x.data_ptr(), w.data_ptr(), None, rstd.data_ptr(), dx.data_ptr(),
                               dw.data_ptr(), None, scratch.data_ptr(), rows, H, _stream()), "rmsnorm_bwd", 2)
    return dx, dw


def _norm_bwd_add(layer, dy, x, w, mean, rstd, add):
    dy, x, w, add = dy.contiguous(), x.contiguous(), w.contiguous(), add.contiguous()
    lib = load()
    lib.jpb_norm_bwd_add.argtypes = [_c_int, _c_int] + [_c_p] * 9 + [_c_int, _c_int, _c_p, _c_p]
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    db = torch.empty_like(w) if layer else None
    rows, H = _rows(x), x.shape[-1]
    scratch = norm_bwd_scratch(rows, H, x.device)
    _check(lib.jpb_norm_bwd_add(layer, _dt(x), dy.data_ptr(), x.data_ptr(), w.data_ptr(), _p(mean), rstd.data_ptr(),
                                dx.data_ptr(), dw.data_ptr(), _p(db), scratch.data_ptr(), rows, H, add.data_ptr(), _stream()),
           "norm_bwd_add", 3 if layer else 2)
    return (dx, dw, db) if layer else (dx, dw)


def rmsnorm_bwd_add(dy, x, w, rstd, add):
    return _norm_bwd_add(0, dy, x, w, None, rstd, add)


def layernorm_bwd_add(dy, x, w, mean, rstd, add):
    return _norm_bwd_add(1, dy, x, w, mean, rstd, add)


def layernorm(x, w, b, eps):
    x = x.contiguous()
    y = torch.empty_like(x)
    mean = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    _check(load().jpb_norm_fwd(1, _dt(x), x.data_ptr(), w.contiguous().data_ptr(), b.contiguous().data_ptr(), y.data_ptr(),
                               mean.data_ptr(), rstd.data_ptr(), _rows(x), x.shape[-1], float(eps), _stream()), "layernorm")
    return y, mean, rstd


def layernorm_bwd(dy, x, w, mean, rstd):
    dy, x, w = dy.contiguous(), x.contiguous(), w.contiguous()
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    rows, H = _rows(x), x.shape[-1]
    scratch = norm_bwd_scratch(rows, H, x.device)
    _check(load().jpb_norm_bwd(1, _dt(x), dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                               dx.data_ptr(), dw.data_ptr(), db.data_ptr(), scratch.data_ptr(), rows, H, _stream()),
           "layernorm_bwd", 3)
    return dx, dw, db


def colsum(dy):
    dy = dy.contiguous()
    rows, cols = _rows(dy), dy.shape[-1]
    out = torch.empty(cols, dtype=dy.dtype, device=dy.device)
    scratch = torch.empty(load().jpb_colsum_scratch_elems(rows, cols), dtype=torch.float32, device=dy.device)
    _check(load().jpb_colsum(_dt(dy), dy.data_ptr(), out.data_ptr(), scratch.data_ptr(), rows, cols, _stream()), "colsum", 2)
    return out


# ---- activations ---------------------------------------------------------------------------------------
def gelu(x):
    x = x.contiguous()
    out = torch.empty_like(x)
    _check(load().jpb_gelu(_dt(x), 0, x.data_ptr(), None, out.data_ptr(), x.numel(), _stream()), "gelu")
    return out


def gelu_bwd(dy, x):
    x, dy = x.contiguous(), dy.contiguous()
    out = torch.empty_like(x)
    _check(load().jpb_gelu(_dt(x), 1, x.data_ptr(), dy.data_ptr(), out.data_ptr(), x.numel(), _stream()), "gelu_bwd")
    return out


def swiglu(gu):
    gu = gu.contiguous()
    F = gu.shape[-1] // 2
    out = torch.empty(*gu.shape[:-1], F, dtype=gu.dtype, device=gu.device)
    _check(load().jpb_swiglu(_dt(gu), 0, gu.data_ptr(), None, out.data_ptr(), _rows(gu), F, _stream()), "swiglu")
    return out


def swiglu_bwd(dy, gu):
    gu, dy = gu.contiguous(), dy.contiguous()
    F = gu.shape[-1] // 2
    out = torch.empty_like(gu)
    _check(load().jpb_swiglu(_dt(gu), 1, gu.data_ptr(), dy.data_ptr(), out.data_ptr(), _rows(gu), F, _stream()), "swiglu_bwd")
    return out


def rope(x, cos, sin, inverse):
    x = x.contiguous()
    B, S, H, D = x.shape
    out = torch.empty_like(x)
    _check(load().jpb_rope(_dt(x), x.data_ptr(), cos.contiguous().data_ptr(), sin.contiguous().data_ptr(), out.data_ptr(),
                           B * S * H, S, H, D, int(inverse), _stream()), "rope")
    return out


def dropout(x, p, seed, offset):
    x = x.contiguous()
    out = torch.empty_like(x)
    lib = load()
    lib.jpb_dropout.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_ll, _c_f, _c_ll, _c_p]
    seed = seed.to(device=x.device, dtype=torch.int64).contiguous()
    _check(lib.jpb_dropout(_dt(x), x.data_ptr(), out.data_ptr(), seed.data_ptr(), int(offset), float(p), x.numel(), _stream()),
           "dropout")
    return out


def _qkv_rope(merge, packed, q, k, v, cos, sin):
    B, S, Hq, D = q.shape
    lib = load()
    lib.jpb_qkv_rope.argtypes = [_c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p]
    cs = None if cos is None else cos.contiguous().data_ptr()
    sn = None if sin is None else sin.contiguous().data_ptr()
    _check(lib.jpb_qkv_rope(_dt(packed), merge, packed.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), cs, sn,
                            B * S, S, Hq, k.shape[2], D, _stream()), "qkv_rope")


def qkv_split(qkv, cos, sin, hq, hkv):
    qkv = qkv.contiguous()
    B, S, _, D = qkv.shape
    q = torch.empty(B, S, hq, D, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(B, S, hkv, D, dtype=qkv.dtype, device=qkv.device)
    v = torch.empty(B, S, hkv, D, dtype=qkv.dtype, device=qkv.device)
    _qkv_rope(0, qkv, q, k, v, cos, sin)
    return q, k, v


def qkv_merge(dq, dk, dv, cos, sin):
    dq, dk, dv = dq.contiguous(), dk.contiguous(), dv.contiguous()
    B, S, Hq, D = dq.shape
    out = torch.empty(B, S, Hq + 2 * dk.shape[2], D, dtype=dq.dtype, device=dq.device)
    _qkv_rope(1, out, dq, dk, dv, cos, sin)
    return out


# ---- embedding / loss / optimizer --------------------------------------------------------------------------
def embedding(ids, table):
    ids = ids.contiguous()
    table = table.contiguous()
    out = torch.empty(*ids.shape, table.shape[1], dtype=table.dtype, device=table.device)
    _check(load().jpb_embedding_fwd(_dt(table), ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.numel(),
                                    table.shape[1], table.shape[0], _stream()), "embedding")
    return out


def embedding_bwd(dy, ids, vocab, out_dtype=None, out: Optional[torch.Tensor] = None, accumulate: bool = False):
    """Gradient of the embedding table: rows of ``dy`` summed by token id.  ``out_dtype`` float32 returns the fp32 sum
    itself (no cast pass); with ``out`` (fp32 [vocab, d]) the rows are added into it (``accumulate``) or it is
    cleared first."""
    dy, ids = dy.contiguous(), ids.contiguous()
    d = dy.shape[-1]
    want = out_dtype or dy.dtype
    if out is not None or want == torch.float32:
        lib = load()
        lib.jpb_embedding_bwd_acc.argtypes = [_c_int, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p]
        acc = out if out is not None else torch.empty(vocab, d, dtype=torch.float32, device=dy.device)
        if acc.dtype != torch.float32 or not acc.is_contiguous():
            raise NativeError("embedding_bwd accumulates into a contiguous float32 table")
        _check(lib.jpb_embedding_bwd_acc(_dt(dy), dy.data_ptr(), ids.data_ptr(), acc.data_ptr(), ids.numel(), d, vocab,
                                         int(not accumulate), _stream()), "embedding_bwd", 1)
        return acc
    acc = torch.empty(vocab, d, dtype=torch.float32, device=dy.device)
    out_t = torch.empty(vocab, d, dtype=dy.dtype, device=dy.device)
    _check(load().jpb_embedding_bwd(_dt(dy), dy.data_ptr(), ids.data_ptr(), acc.data_ptr(), out_t.data_ptr(), ids.numel(), d,
                                    vocab, _stream()), "embedding_bwd", 2)
    return out_t


def cross_entropy(logits, labels):
    logits, labels = logits.contiguous(), labels.contiguous()
    rows, V = _rows(logits), logits.shape[-1]
    loss = torch.empty(logits.shape[:-1], dtype=torch.float32, device=logits.device)
    lse = torch.empty_like(loss)
    _check(load().jpb_ce_fwd(_dt(logits), logits.data_ptr(), labels.data_ptr(), loss.data_ptr(), lse.data_ptr(), rows, V,
                             _stream()), "cross_entropy")
    return loss, lse


def cross_entropy_bwd(dloss, logits, labels, lse):
    logits, labels = logits.contiguous(), labels.contiguous()
    dloss = dloss.contiguous().float()
    rows, V = _rows(logits), logits.shape[-1]
    out = torch.empty_like(logits)
    _check(load().jpb_ce_bwd(_dt(logits), dloss.data_ptr(), logits.data_ptr(), labels.data_ptr(), lse.contiguous().data_ptr(),
                             out.data_ptr(), rows, V, _stream()), "cross_entropy_bwd")
    return out


def adamw(master, grad, m, v, step, lr, beta1, beta2, eps, weight_decay, grad_scale, out_dtype, lp_old=None,
          inplace=False):
    grad = grad.contiguous()
    if inplace:
        if not (master.is_contiguous() and m.is_contiguous() and v.is_contiguous()):
            raise NativeError("in-place adamw needs contiguous state tensors")
        p2, m2, v2 = master, m, v
        reuse = lp_old is not None and lp_old.dtype == out_dtype and lp_old.is_contiguous()
        lp = lp_old if reuse else torch.empty(master.shape, dtype=out_dtype, device=master.device)
    else:
        master, m, v = master.contiguous(), m.contiguous(), v.contiguous()
        p2, m2, v2 = torch.empty_like(master), torch.empty_like(m), torch.empty_like(v)
        lp = torch.empty(master.shape, dtype=out_dtype, device=master.device)
    step = step.to(device=master.device, dtype=torch.int64)
    out_code = 0 if out_dtype == torch.float32 else 1
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise NativeError(f"adamw low-precision copy must be float32 or bfloat16, got {out_dtype}")
    _check(load().jpb_adamw(_dt(grad), out_code, master.data_ptr(), grad.data_ptr(), m.data_ptr(), v.data_ptr(),
                            step.data_ptr(), p2.data_ptr(), m2.data_ptr(), v2.data_ptr(), lp.data_ptr(), master.numel(),
                            float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), float(grad_scale),
                            _stream()), "adamw")
    return p2, m2, v2, lp


# ---- attention: bound in attention.py once the kernel library provides it ----------------------------------
def attention(q, k, v, causal, scale):
    from . import attention as att

    return att.attention_fwd(q, k, v, causal, scale)


def attention_bwd(do, q, k, v, o, lse, causal, scale):
    from . import attention as att

    return att.attention_bwd(do, q, k, v, o, lse, causal, scale)
