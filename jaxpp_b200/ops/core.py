"""The closed set of tensor ops that captured train steps are made of.

Every op is a ``torch.library`` custom op in the ``b200`` namespace with

* a shape function (``register_fake``) so a train step can be traced without data,
* a reference implementation in plain PyTorch (runs on CPU, and on CUDA only when native
  kernels are switched off with ``JAXPP_B200_NATIVE=0``),
* a native sm_100a implementation (``jaxpp_b200.ops.native``) used for CUDA tensors, and
* an explicit backward written in terms of other ``b200`` ops, with the input-gradient and
  weight-gradient parts as *separate* ops so that the compiler can split a backward task into
  its activation half and its weight half by dataflow (zero-bubble schedules).

The reference framework has no op layer of its own: these computations are XLA fusions of the
user's jnp code there (e.g. examples/basic.py:33-91 for dense/attention/LayerNorm/GELU).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from ..utils import config

_lib = torch.library.Library("b200", "DEF")

_NATIVE = None

# op overload -> the Python function registered as its implementation.  Generated task code calls these directly
# instead of going through ``torch.ops`` (the dispatcher costs about 10 us per call of a Python-implemented op, which
# is the whole budget of a small kernel); eager calls and tracing still use the registered ops.
DIRECT: dict = {}


def _native():
    """The native kernel module; raises if it cannot be loaded (no silent fallback on CUDA)."""
    global _NATIVE
    if _NATIVE is None:
        from . import native

        native.load()
        _NATIVE = native
    return _NATIVE


def _use_native(t: Tensor) -> bool:
    return t.is_cuda and config.use_native_kernels.value


def _define(schema: str, ref_impl, fake_impl, native_name: str | None = None):
    """Register ``b200::<schema>`` with reference, fake and (optional) native implementations."""
    name = schema.split("(")[0]
    _lib.define(schema)
    qual = f"b200::{name}"

    if native_name is None:
        impl = ref_impl
    else:
        def impl(*args, __ref=ref_impl, __nn=native_name):
            first = next(a for a in args if isinstance(a, Tensor))
            if _use_native(first):
                return getattr(_native(), __nn)(*args)
            return __ref(*args)

    _lib.impl(name, impl, "CompositeExplicitAutograd")
    torch.library.register_fake(qual, fake_impl)
    DIRECT[getattr(torch.ops.b200, name).default] = impl
    return getattr(torch.ops.b200, name)


def _autograd(name: str, backward, setup_context):
    torch.library.register_autograd(f"b200::{name}", backward, setup_context=setup_context)


def _f32(t: Tensor) -> Tensor:
    return t.float()


# ======================================================================================
# linear:  y[..., N] = x[..., K] @ w[N, K]^T (+ bias[N])
# ======================================================================================

def _linear_ref(x, w, bias):
    y = x @ w.t()
    return y if bias is None else y + bias


def _linear_fake(x, w, bias):
    return x.new_empty(*x.shape[:-1], w.shape[0])


linear = _define("linear(Tensor x, Tensor w, Tensor? bias) -> Tensor", _linear_ref, _linear_fake, "linear")


def _linear_dgrad_ref(dy, w):
    return dy @ w


linear_dgrad = _define(
    "linear_dgrad(Tensor dy, Tensor w) -> Tensor",
    _linear_dgrad_ref,
    lambda dy, w: dy.new_empty(*dy.shape[:-1], w.shape[1]),
    "linear_dgrad",
)


# dtype of weight gradients produced by the backward of ``linear`` (None = same as the activations).
# Set to torch.float32 to get fp32 main gradients straight out of the GEMM epilogue.
WGRAD_DTYPE: list = [None]


def _linear_wgrad_ref(dy, x, out_dtype=None):
    out = dy.reshape(-1, dy.shape[-1]).float().t() @ x.reshape(-1, x.shape[-1]).float()
    return out.to(out_dtype if out_dtype is not None else dy.dtype)


def _linear_wgrad_native_or_ref(dy, x, out_dtype=None):
    if _use_native(dy):
        nat = _native()
        if out_dtype is None or out_dtype == dy.dtype:
            return nat.linear_wgrad(dy, x)
        if out_dtype != torch.float32:
            raise RuntimeError(f"linear_wgrad writes bfloat16 or float32, not {out_dtype}")
        out = torch.empty(dy.shape[-1], x.shape[-1], dtype=torch.float32, device=dy.device)
        return nat.linear_wgrad(dy, x, out=out)
    return _linear_wgrad_ref(dy, x, out_dtype)


_lib.define("linear_wgrad(Tensor dy, Tensor x, ScalarType? out_dtype=None) -> Tensor")
_lib.impl("linear_wgrad", _linear_wgrad_native_or_ref, "CompositeExplicitAutograd")
torch.library.register_fake(
    "b200::linear_wgrad",
    lambda dy, x, out_dtype=None: dy.new_empty(dy.shape[-1], x.shape[-1], dtype=out_dtype or dy.dtype),
)
linear_wgrad = torch.ops.b200.linear_wgrad
DIRECT[linear_wgrad.default] = _linear_wgrad_native_or_ref

# column sums, used for bias gradients
colsum = _define(
    "colsum(Tensor dy) -> Tensor",
    lambda dy: dy.reshape(-1, dy.shape[-1]).float().sum(0).to(dy.dtype),
    lambda dy: dy.new_empty(dy.shape[-1]),
    "colsum",
)


def _linear_setup(ctx, inputs, output):
    x, w, bias = inputs
    ctx.save_for_backward(x, w)
    ctx.has_bias = bias is not None


def _linear_bwd(ctx, dy):
    x, w = ctx.saved_tensors
    dx = linear_dgrad(dy, w) if ctx.needs_input_grad[0] else None
    dw = linear_wgrad(dy, x, WGRAD_DTYPE[0]) if ctx.needs_input_grad[1] else None
    db = colsum(dy) if ctx.has_bias and ctx.needs_input_grad[2] else None
    return dx, dw, db


_autograd("linear", _linear_bwd, _linear_setup)


# ======================================================================================
# grouped linear (equal-sized groups: the local experts of a mixture-of-experts layer)
#   y[e] = x[e] @ w[e]^T   x [E, M, K], w [E, N, K] -> [E, M, N]; one launch on the GPU
# ======================================================================================

def _wg_dtype(dy, out_dtype):
    return out_dtype if out_dtype is not None else dy.dtype


# ``counts`` ([E, M / seg_rows] int32) describes groups of unequal size inside the equal-sized storage: the M rows of a
# group are segments of ``seg_rows`` rows, and only the first counts[e, s] rows of segment s hold data; the caller
# guarantees that the others are zero.  The results do not depend on it (zero rows give zero products), so the
# references ignore it; the GPU kernels skip the tiles and reduction blocks that hold no data.
linear_batched = _define(
    "linear_batched(Tensor x, Tensor w, Tensor? counts=None, int seg_rows=0) -> Tensor",
    lambda x, w, counts=None, seg_rows=0: torch.bmm(x, w.transpose(1, 2)),
    lambda x, w, counts=None, seg_rows=0: x.new_empty(x.shape[0], x.shape[1], w.shape[1]),
    "linear_batched",
)
linear_dgrad_batched = _define(
    "linear_dgrad_batched(Tensor dy, Tensor w, Tensor? counts=None, int seg_rows=0) -> Tensor",
    lambda dy, w, counts=None, seg_rows=0: torch.bmm(dy, w),
    lambda dy, w, counts=None, seg_rows=0: dy.new_empty(dy.shape[0], dy.shape[1], w.shape[2]),
    "linear_dgrad_batched",
)
linear_wgrad_batched = _define(
    "linear_wgrad_batched(Tensor dy, Tensor x, ScalarType? out_dtype=None, Tensor? counts=None, int seg_rows=0) -> Tensor",
    lambda dy, x, out_dtype=None, counts=None, seg_rows=0:
        torch.bmm(_f32(dy).transpose(1, 2), _f32(x)).to(_wg_dtype(dy, out_dtype)),
    lambda dy, x, out_dtype=None, counts=None, seg_rows=0:
        dy.new_empty(dy.shape[0], dy.shape[2], x.shape[2], dtype=_wg_dtype(dy, out_dtype)),
    "linear_wgrad_batched",
)


def _linear_batched_setup(ctx, inputs, output):
    x, w, counts, ctx.seg_rows = inputs
    ctx.has_counts = counts is not None
    ctx.save_for_backward(*([x, w] + ([counts] if ctx.has_counts else [])))


def _linear_batched_bwd(ctx, dy):
    x, w = ctx.saved_tensors[:2]
    counts = ctx.saved_tensors[2] if ctx.has_counts else None
    dy = dy.contiguous()
    dx = linear_dgrad_batched(dy, w, counts, ctx.seg_rows) if ctx.needs_input_grad[0] else None
    dw = linear_wgrad_batched(dy, x, WGRAD_DTYPE[0], counts, ctx.seg_rows) if ctx.needs_input_grad[1] else None
    return dx, dw, None, None


_autograd("linear_batched", _linear_batched_bwd, _linear_batched_setup)


# ======================================================================================
# RMSNorm / LayerNorm (statistics in fp32)
# ======================================================================================

def _rmsnorm_ref(x, w, eps):
    xf = _f32(x)
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * _f32(w)).to(x.dtype), rstd.squeeze(-1)


rmsnorm = _define(
    "rmsnorm(Tensor x, Tensor w, float eps) -> (Tensor, Tensor)",
    _rmsnorm_ref,
    lambda x, w, eps: (torch.empty_like(x), x.new_empty(x.shape[:-1], dtype=torch.float32)),
    "rmsnorm",
)


def _rmsnorm_bwd_ref(dy, x, w, rstd):
    xf, dyf, wf = _f32(x), _f32(dy), _f32(w)
    xhat = xf * rstd.unsqueeze(-1)
    g = dyf * wf
    dx = (g - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd.unsqueeze(-1)
    dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
    return dx.to(x.dtype), dw.to(w.dtype)


rmsnorm_bwd = _define(
    "rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd) -> (Tensor, Tensor)",
    _rmsnorm_bwd_ref,
    lambda dy, x, w, rstd: (torch.empty_like(x), torch.empty_like(w)),
    "rmsnorm_bwd",
)


def _rmsnorm_bwd_add_ref(dy, x, w, rstd, add):
    dx, dw = _rmsnorm_bwd_ref(dy, x, w, rstd)
    return dx + add, dw


# dx + (gradient arriving over the residual connection) in the pass that produces dx; the graph rewrite in
# compiler/peephole.py puts it in place of ``rmsnorm_bwd`` followed by ``add``
rmsnorm_bwd_add = _define(
    "rmsnorm_bwd_add(Tensor dy, Tensor x, Tensor w, Tensor rstd, Tensor add) -> (Tensor, Tensor)",
    _rmsnorm_bwd_add_ref,
    lambda dy, x, w, rstd, add: (torch.empty_like(x), torch.empty_like(w)),
    "rmsnorm_bwd_add",
)


def _rmsnorm_setup(ctx, inputs, output):
    x, w, _ = inputs
    ctx.save_for_backward(x, w, output[1])


def _rmsnorm_autograd(ctx, dy, _drstd):
    x, w, rstd = ctx.saved_tensors
    dx, dw = rmsnorm_bwd(dy, x, w, rstd)
    return dx, dw, None


_autograd("rmsnorm", _rmsnorm_autograd, _rmsnorm_setup)


def _layernorm_ref(x, w, b, eps):
    xf = _f32(x)
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).pow(2).mean(-1, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean) * rstd * _f32(w) + _f32(b)
    return y.to(x.dtype), mean.squeeze(-1), rstd.squeeze(-1)


layernorm = _define(
    "layernorm(Tensor x, Tensor w, Tensor b, float eps) -> (Tensor, Tensor, Tensor)",
    _layernorm_ref,
    lambda x, w, b, eps: (
        torch.empty_like(x),
        x.new_empty(x.shape[:-1], dtype=torch.float32),
        x.new_empty(x.shape[:-1], dtype=torch.float32),
    ),
    "layernorm",
)


def _layernorm_bwd_ref(dy, x, w, mean, rstd):
    xf, dyf, wf = _f32(x), _f32(dy), _f32(w)
    xhat = (xf - mean.unsqueeze(-1)) * rstd.unsqueeze(-1)
    g = dyf * wf
    dx = (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd.unsqueeze(-1)
    dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
    db = dyf.reshape(-1, x.shape[-1]).sum(0)
    return dx.to(x.dtype), dw.to(w.dtype), db.to(w.dtype)


layernorm_bwd = _define(
    "layernorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor mean, Tensor rstd) -> (Tensor, Tensor, Tensor)",
    _layernorm_bwd_ref,
    lambda dy, x, w, mean, rstd: (torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)),
    "layernorm_bwd",
)


def _layernorm_bwd_add_ref(dy, x, w, mean, rstd, add):
    dx, dw, db = _layernorm_bwd_ref(dy, x, w, mean, rstd)
    return dx + add, dw, db


layernorm_bwd_add = _define(
    "layernorm_bwd_add(Tensor dy, Tensor x, Tensor w, Tensor mean, Tensor rstd, Tensor add) -> (Tensor, Tensor, Tensor)",
    _layernorm_bwd_add_ref,
    lambda dy, x, w, mean, rstd, add: (torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)),
    "layernorm_bwd_add",
)


def _layernorm_setup(ctx, inputs, output):
    x, w, b, _ = inputs
    ctx.save_for_backward(x, w, output[1], output[2])


def _layernorm_autograd(ctx, dy, _dm, _dr):
    x, w, mean, rstd = ctx.saved_tensors
    dx, dw, db = layernorm_bwd(dy, x, w, mean, rstd)
    return dx, dw, db, None


_autograd("layernorm", _layernorm_autograd, _layernorm_setup)


# ======================================================================================
# Activations: GELU (tanh approximation) and SwiGLU on a fused [gate | up] tensor
# ======================================================================================
_K0 = math.sqrt(2.0 / math.pi)
_K1 = 0.044715


def _gelu_ref(x):
    xf = _f32(x)
    return (0.5 * xf * (1.0 + torch.tanh(_K0 * (xf + _K1 * xf.pow(3))))).to(x.dtype)


def _gelu_bwd_ref(dy, x):
    xf = _f32(x)
    t = torch.tanh(_K0 * (xf + _K1 * xf.pow(3)))
    dt = (1.0 - t * t) * _K0 * (1.0 + 3.0 * _K1 * xf * xf)
    return (_f32(dy) * (0.5 * (1.0 + t) + 0.5 * xf * dt)).to(x.dtype)


gelu = _define("gelu(Tensor x) -> Tensor", _gelu_ref, lambda x: torch.empty_like(x), "gelu")
gelu_bwd = _define("gelu_bwd(Tensor dy, Tensor x) -> Tensor", _gelu_bwd_ref, lambda dy, x: torch.empty_like(x), "gelu_bwd")
_autograd(
    "gelu",
    lambda ctx, dy: gelu_bwd(dy, ctx.saved_tensors[0]),
    lambda ctx, inputs, output: ctx.save_for_backward(inputs[0]),
)


# ======================================================================================
# dropout with a counter-based generator: the mask is a function of (seed, offset, element index), so backward
# regenerates it and a pipelined run draws the same numbers as the sequential one (the reference keeps
# threefry keys with the same property, tests/functional_testing/test_dropout_enabled.py:55)
# ======================================================================================
_M32 = 0xFFFFFFFF


def _mul32(a: int, b: Tensor):
    """(hi, lo) 32-bit halves of a * b for a 32-bit constant ``a`` and int64 ``b`` holding 32-bit values."""
    t, u = a * (b & 0xFFFF), a * (b >> 16)
    low = ((u & 0xFFFF) << 16) + (t & _M32)
    return ((u >> 16) + (t >> 32) + (low >> 32)) & _M32, low & _M32


def philox_u32(n_blocks: int, seed: Tensor, offset: int, device) -> Tensor:
    """[n_blocks, 4] int64 tensor of the 32-bit outputs of Philox4x32-10 at counters (block, offset), key ``seed``."""
    q = torch.arange(n_blocks, dtype=torch.int64, device=device)
    c0, c1 = q & _M32, (q >> 32) & _M32
    c2 = torch.full_like(q, offset & _M32)
    c3 = torch.full_like(q, (offset >> 32) & _M32)
    seed = seed.to(device=device, dtype=torch.int64)
    k0, k1 = (seed & _M32).expand_as(q).clone(), ((seed >> 32) & _M32).expand_as(q).clone()
    for _ in range(10):
        hi0, lo0 = _mul32(0xD2511F53, c0)
        hi1, lo1 = _mul32(0xCD9E8D57, c2)
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0, k1 = (k0 + 0x9E3779B9) & _M32, (k1 + 0xBB67AE85) & _M32
    return torch.stack([c0, c1, c2, c3], dim=1)


def _dropout_ref(x, p, seed, offset):
    n = x.numel()
    words = philox_u32((n + 3) // 4, seed, offset, x.device).reshape(-1)[:n].view(x.shape)
    t = p * 4294967296.0
    threshold = 0xFFFFFFFF if t >= 4294967295.0 else int(t)
    keep = words >= threshold
    return torch.where(keep, _f32(x) * (1.0 / (1.0 - p)), torch.zeros((), device=x.device)).to(x.dtype)


dropout = _define(
    "dropout(Tensor x, float p, Tensor seed, int offset) -> Tensor",
    _dropout_ref, lambda x, p, seed, offset: torch.empty_like(x), "dropout",
)


def _dropout_setup(ctx, inputs, output):
    _, ctx.p, seed, ctx.offset = inputs
    ctx.save_for_backward(seed)


_autograd("dropout", lambda ctx, dy: (dropout(dy.contiguous(), ctx.p, ctx.saved_tensors[0], ctx.offset), None, None, None),
          _dropout_setup)


def _swiglu_ref(gu):
    g, u = _f32(gu).chunk(2, dim=-1)
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def _swiglu_bwd_ref(dy, gu):
    g, u = _f32(gu).chunk(2, dim=-1)
    s = torch.sigmoid(g)
    dyf = _f32(dy)
    dg = dyf * u * s * (1.0 + g * (1.0 - s))
    du = dyf * g * s
    return torch.cat([dg, du], dim=-1).to(gu.dtype)


swiglu = _define(
    "swiglu(Tensor gate_up) -> Tensor",
    _swiglu_ref,
    lambda gu: gu.new_empty(*gu.shape[:-1], gu.shape[-1] // 2),
    "swiglu",
)
swiglu_bwd = _define(
    "swiglu_bwd(Tensor dy, Tensor gate_up) -> Tensor", _swiglu_bwd_ref, lambda dy, gu: torch.empty_like(gu), "swiglu_bwd"
)
_autograd(
    "swiglu",
    lambda ctx, dy: swiglu_bwd(dy, ctx.saved_tensors[0]),
    lambda ctx, inputs, output: ctx.save_for_backward(inputs[0]),
)


# ======================================================================================
# RoPE on [B, S, H, D] with half-split rotation (Llama convention); cos/sin are [S, D/2] fp32
# ======================================================================================

def _rope_ref(x, cos, sin, inverse):
    xf = _f32(x)
    d2 = x.shape[-1] // 2
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c = cos[None, :, None, :]
    s = -sin[None, :, None, :] if inverse else sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


rope = _define(
    "rope(Tensor x, Tensor cos, Tensor sin, bool inverse) -> Tensor",
    _rope_ref,
    lambda x, cos, sin, inverse: torch.empty_like(x),
    "rope",
)


def _rope_setup(ctx, inputs, output):
    _, cos, sin, inverse = inputs
    ctx.save_for_backward(cos, sin)
    ctx.inverse = inverse


def _rope_autograd(ctx, dy):
    cos, sin = ctx.saved_tensors
    return rope(dy, cos, sin, not ctx.inverse), None, None, None


_autograd("rope", _rope_autograd, _rope_setup)


# ======================================================================================
# qkv_split: packed projection [B, S, Hq + 2*Hkv, D] -> contiguous q [B,S,Hq,D], k, v [B,S,Hkv,D] with RoPE on
# q and k (cos/sin None: plain split); qkv_merge is its transpose (inverse rotation) and its backward
# ======================================================================================

def _qkv_split_ref(qkv, cos, sin, hq, hkv):
    q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
    if cos is not None:
        q, k = _rope_ref(q, cos, sin, False), _rope_ref(k, cos, sin, False)
    return q.contiguous(), k.contiguous(), v.contiguous()


def _qkv_merge_ref(dq, dk, dv, cos, sin):
    if cos is not None:
        dq, dk = _rope_ref(dq, cos, sin, True), _rope_ref(dk, cos, sin, True)
    return torch.cat([dq, dk, dv], dim=2)


def _qkv_split_fake(qkv, cos, sin, hq, hkv):
    B, S, _, D = qkv.shape
    return qkv.new_empty(B, S, hq, D), qkv.new_empty(B, S, hkv, D), qkv.new_empty(B, S, hkv, D)


qkv_split = _define(
    "qkv_split(Tensor qkv, Tensor? cos, Tensor? sin, int hq, int hkv) -> (Tensor, Tensor, Tensor)",
    _qkv_split_ref, _qkv_split_fake, "qkv_split",
)
qkv_merge = _define(
    "qkv_merge(Tensor dq, Tensor dk, Tensor dv, Tensor? cos, Tensor? sin) -> Tensor",
    _qkv_merge_ref,
    lambda dq, dk, dv, cos, sin: dq.new_empty(dq.shape[0], dq.shape[1], dq.shape[2] + 2 * dk.shape[2], dq.shape[3]),
    "qkv_merge",
)


def _qkv_split_setup(ctx, inputs, output):
    _, cos, sin, ctx.hq, ctx.hkv = inputs
    ctx.has_rope = cos is not None
    if ctx.has_rope:
        ctx.save_for_backward(cos, sin)


def _qkv_split_bwd(ctx, dq, dk, dv):
    cos, sin = ctx.saved_tensors if ctx.has_rope else (None, None)
    return qkv_merge(dq.contiguous(), dk.contiguous(), dv.contiguous(), cos, sin), None, None, None, None


def _qkv_merge_setup(ctx, inputs, output):
    dq, dk, _, cos, sin = inputs
    ctx.hq, ctx.hkv = dq.shape[2], dk.shape[2]
    ctx.has_rope = cos is not None
    if ctx.has_rope:
        ctx.save_for_backward(cos, sin)


def _qkv_merge_bwd(ctx, g):
    cos, sin = ctx.saved_tensors if ctx.has_rope else (None, None)
    q, k, v = qkv_split(g.contiguous(), cos, sin, ctx.hq, ctx.hkv)
    return q, k, v, None, None


_autograd("qkv_split", _qkv_split_bwd, _qkv_split_setup)
_autograd("qkv_merge", _qkv_merge_bwd, _qkv_merge_setup)


# ======================================================================================
# Attention on [B, S, H, D] (q) and [B, S, Hkv, D] (k, v); returns output and log-sum-exp
# ======================================================================================

def _attn_ref(q, k, v, causal, scale):
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    rep = H // Hkv
    qf = _f32(q).permute(0, 2, 1, 3)
    kf = _f32(k).permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = _f32(v).permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        Sk = k.shape[1]
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(Sk - S)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = (p @ vf).permute(0, 2, 1, 3)
    return o.to(q.dtype).contiguous(), lse  # lse: [B, H, S] fp32


attention = _define(
    "attention(Tensor q, Tensor k, Tensor v, bool causal, float scale) -> (Tensor, Tensor)",
    _attn_ref,
    lambda q, k, v, causal, scale: (
        torch.empty_like(q),
        q.new_empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32),
    ),
    "attention",
)


def _attn_bwd_ref(do, q, k, v, o, lse, causal, scale):
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    rep = H // Hkv
    qf = _f32(q).permute(0, 2, 1, 3)
    kf = _f32(k).permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = _f32(v).permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    dof = _f32(do).permute(0, 2, 1, 3)
    of = _f32(o).permute(0, 2, 1, 3)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        Sk = k.shape[1]
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(Sk - S)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = p.transpose(-1, -2) @ dof
    dp = dof @ vf.transpose(-1, -2)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kf
    dk = ds.transpose(-1, -2) @ qf
    if rep > 1:
        dk = dk.reshape(B, Hkv, rep, k.shape[1], D).sum(2)
        dv = dv.reshape(B, Hkv, rep, k.shape[1], D).sum(2)
    to = lambda t, like: t.permute(0, 2, 1, 3).to(like.dtype).contiguous()
    return to(dq, q), to(dk, k), to(dv, v)


attention_bwd = _define(
    "attention_bwd(Tensor do, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, bool causal, float scale)"
    " -> (Tensor, Tensor, Tensor)",
    _attn_bwd_ref,
    lambda do, q, k, v, o, lse, causal, scale: (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)),
    "attention_bwd",
)


def _attn_setup(ctx, inputs, output):
    q, k, v, causal, scale = inputs
    ctx.save_for_backward(q, k, v, output[0], output[1])
    ctx.causal, ctx.scale = causal, scale


def _attn_autograd(ctx, do, _dlse):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = attention_bwd(do, q, k, v, o, lse, ctx.causal, ctx.scale)
    return dq, dk, dv, None, None


_autograd("attention", _attn_autograd, _attn_setup)


# ======================================================================================
# Cross entropy over the last dim: returns per-row loss (fp32) and log-sum-exp (fp32)
# ======================================================================================

def _ce_ref(logits, labels):
    lf = _f32(logits)
    lse = torch.logsumexp(lf, dim=-1)
    picked = lf.gather(-1, labels.unsqueeze(-1)).squeeze(-1)
    return lse - picked, lse


cross_entropy = _define(
    "cross_entropy(Tensor logits, Tensor labels) -> (Tensor, Tensor)",
    _ce_ref,
    lambda logits, labels: (
        logits.new_empty(logits.shape[:-1], dtype=torch.float32),
        logits.new_empty(logits.shape[:-1], dtype=torch.float32),
    ),
    "cross_entropy",
)


def _ce_bwd_ref(dloss, logits, labels, lse):
    p = torch.exp(_f32(logits) - lse.unsqueeze(-1))
    p.scatter_add_(-1, labels.unsqueeze(-1), -torch.ones_like(p[..., :1]))
    return (p * dloss.unsqueeze(-1)).to(logits.dtype)


cross_entropy_bwd = _define(
    "cross_entropy_bwd(Tensor dloss, Tensor logits, Tensor labels, Tensor lse) -> Tensor",
    _ce_bwd_ref,
    lambda dloss, logits, labels, lse: torch.empty_like(logits),
    "cross_entropy_bwd",
)


def _ce_setup(ctx, inputs, output):
    logits, labels = inputs
    ctx.save_for_backward(logits, labels, output[1])


def _ce_autograd(ctx, dloss, _dlse):
    logits, labels, lse = ctx.saved_tensors
    return cross_entropy_bwd(dloss.contiguous(), logits, labels, lse), None


_autograd("cross_entropy", _ce_autograd, _ce_setup)


# ======================================================================================
# Embedding gather / scatter-add
# ======================================================================================
embedding = _define(
    "embedding(Tensor ids, Tensor table) -> Tensor",
    lambda ids, table: table[ids],
    lambda ids, table: table.new_empty(*ids.shape, table.shape[1]),
    "embedding",
)


def _emb_bwd_ref(dy, ids, vocab, out_dtype=None):
    out = torch.zeros(vocab, dy.shape[-1], dtype=torch.float32, device=dy.device)
    out.index_add_(0, ids.reshape(-1), _f32(dy).reshape(-1, dy.shape[-1]))
    return out.to(out_dtype if out_dtype is not None else dy.dtype)


# ``out_dtype`` float32 (what ``WGRAD_DTYPE`` asks for) returns the fp32 sum without a cast pass, and makes the op a
# weight-gradient sink: inside a microbatch loop it adds straight into the accumulator (ops/sink.py)
embedding_bwd = _define(
    "embedding_bwd(Tensor dy, Tensor ids, int vocab, ScalarType? out_dtype=None) -> Tensor",
    _emb_bwd_ref,
    lambda dy, ids, vocab, out_dtype=None: dy.new_empty(vocab, dy.shape[-1], dtype=out_dtype or dy.dtype),
    "embedding_bwd",
)


def _emb_setup(ctx, inputs, output):
    ids, table = inputs
    ctx.save_for_backward(ids)
    ctx.vocab = table.shape[0]


_autograd("embedding",
          lambda ctx, dy: (None, embedding_bwd(dy.contiguous(), ctx.saved_tensors[0], ctx.vocab, WGRAD_DTYPE[0])), _emb_setup)


# ======================================================================================
# Fused AdamW step (functional): returns new (master, m, v, low-precision copy)
# ``master``/``m``/``v`` are fp32; ``grad`` may be bf16 or fp32; ``step`` is a 0-d tensor (1-based)
# ======================================================================================

def _adamw_ref(master, grad, m, v, step, lr, beta1, beta2, eps, weight_decay, grad_scale, out_dtype, lp_old=None,
               inplace=False):
    g = _f32(grad) * grad_scale
    m2 = beta1 * m + (1.0 - beta1) * g
    v2 = beta2 * v + (1.0 - beta2) * g * g
    t = step.to(torch.float32)
    bc1 = 1.0 - beta1 ** t
    bc2 = 1.0 - beta2 ** t
    upd = (m2 / bc1) / ((v2 / bc2).sqrt() + eps)
    p2 = master * (1.0 - lr * weight_decay) - lr * upd
    if inplace:  # the caller gives up the old state: reuse its storage
        master.copy_(p2), m.copy_(m2), v.copy_(v2)
        lp = lp_old.copy_(p2) if lp_old is not None and lp_old.dtype == out_dtype else p2.to(out_dtype)
        return master, m, v, lp
    return p2, m2, v2, p2.to(out_dtype)


adamw = _define(
    "adamw(Tensor master, Tensor grad, Tensor m, Tensor v, Tensor step, float lr, float beta1, float beta2,"
    " float eps, float weight_decay, float grad_scale, ScalarType out_dtype, Tensor? lp_old=None, bool inplace=False)"
    " -> (Tensor, Tensor, Tensor, Tensor)",
    _adamw_ref,
    lambda master, grad, m, v, step, lr, b1, b2, eps, wd, gs, out_dtype, lp_old=None, inplace=False: (
        torch.empty_like(master),
        torch.empty_like(m),
        torch.empty_like(v),
        master.new_empty(master.shape, dtype=out_dtype),
    ),
    "adamw",
)


# ======================================================================================
# Mean-squared-error helper used by the encoder example (kept as ATen: it is glue, not hot)
# ======================================================================================

def mse_loss(out: Tensor, target: Tensor) -> Tensor:
    return (out.float() - target.float()).pow(2).mean()


__all__ = [
    "linear", "linear_dgrad", "linear_wgrad", "colsum", "rmsnorm", "rmsnorm_bwd", "layernorm", "layernorm_bwd",
    "gelu", "gelu_bwd", "swiglu", "swiglu_bwd", "rope", "attention", "attention_bwd", "cross_entropy",
    "cross_entropy_bwd", "embedding", "embedding_bwd", "adamw", "mse_loss",
]
