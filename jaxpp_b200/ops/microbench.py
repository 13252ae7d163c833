"""Run one native kernel on one shape, timed with CUDA events — the small cases used for profiling.

    python -m jaxpp_b200.ops.microbench gemm --m 8192 --n 8192 --k 8192 --layout fwd --iters 5
    python -m jaxpp_b200.ops.microbench attn_fwd --batch 2 --seq 4096 --heads 16 --head-dim 128
    python -m jaxpp_b200.ops.microbench rmsnorm --rows 32768 --hidden 4096

Prints one JSON line with the median time, the achieved TFLOP/s or GB/s and the fraction of the measured
peak (``MEASURED_PEAKS.json`` at the repository root if present, else 1412 TFLOP/s / 6542 GB/s).  Between
timed iterations a 256 MiB buffer is overwritten to flush L2.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os

import torch

from . import attention as att
from . import native


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        p = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        return float(p["bf16_tflops"]), float(p["hbm_gbs"])
    except Exception:
        return 1590.0, 6650.0


def timed(fn, iters: int, warmup: int = 3, flush: bool = True) -> float:
    buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def suite(rows: int, hidden: int, iters: int, warmup: int, flush: bool):
    """Every memory-bound kernel of the library once per iteration on inputs larger than L2, one JSON line each:
    algorithmic bytes (what the op must read and write), CUDA-event time, GB/s and the fraction of the measured copy
    bandwidth.  With ``--iters 1 --warmup 0`` every kernel launches once, which is the form to put under a profiler."""
    from ..parallel import moe  # noqa: F401  (registers the router op)

    _, bw_peak = _peaks()
    bf = torch.bfloat16
    R, H = rows, hidden
    x, dy = torch.randn(R, H, device="cuda", dtype=bf), torch.randn(R, H, device="cuda", dtype=bf)
    w, b = torch.randn(H, device="cuda", dtype=bf), torch.randn(H, device="cuda", dtype=bf)
    _, rstd = native.rmsnorm(x, w, 1e-5)
    _, mean, lrstd = native.layernorm(x, w, b, 1e-5)
    gu = torch.randn(R, 2 * H, device="cuda", dtype=bf)
    dyf = torch.randn(R, H, device="cuda", dtype=bf)
    B, S, Hq, Hkv, D = max(1, R // 4096), 4096, 32, 32, 128
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda", dtype=bf)
    pos = torch.arange(S, device="cuda", dtype=torch.float32)[:, None] * torch.rand(D // 2, device="cuda")[None, :]
    cos, sin = pos.cos().contiguous(), pos.sin().contiguous()
    q, k, v = native.qkv_split(qkv, cos, sin, Hq, Hkv)
    V = 32000
    Rl = max(1024, R // 4)
    logits = torch.randn(Rl, V, device="cuda", dtype=bf)
    labels = torch.randint(0, V, (Rl,), device="cuda")
    _, lse = native.cross_entropy(logits, labels)
    dloss = torch.ones(Rl, device="cuda")
    table = torch.randn(V, H, device="cuda", dtype=bf)
    ids = torch.randint(0, V, (R,), device="cuda")
    n = R * H
    pm, pg = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m_, v_ = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    step = torch.ones((), dtype=torch.int64, device="cuda")
    seed = torch.tensor(1234, dtype=torch.int64, device="cuda")
    rl = torch.randn(R * 8, 8, device="cuda")
    e2 = 2
    cases = [
        ("rmsnorm", 2 * n * e2, lambda: native.rmsnorm(x, w, 1e-5)),
        ("rmsnorm_bwd", 3 * n * e2, lambda: native.rmsnorm_bwd(dy, x, w, rstd)),
        ("rmsnorm_bwd_add", 4 * n * e2, lambda: native.rmsnorm_bwd_add(dy, x, w, rstd, dyf)),
        ("layernorm", 2 * n * e2, lambda: native.layernorm(x, w, b, 1e-5)),
        ("layernorm_bwd", 3 * n * e2, lambda: native.layernorm_bwd(dy, x, w, mean, lrstd)),
        ("swiglu", 3 * n * e2, lambda: native.swiglu(gu)),
        ("swiglu_bwd", 5 * n * e2, lambda: native.swiglu_bwd(dyf, gu)),
        ("gelu", 2 * n * e2, lambda: native.gelu(x)),
        ("gelu_bwd", 3 * n * e2, lambda: native.gelu_bwd(dy, x)),
        ("qkv_split_rope", 2 * qkv.numel() * e2, lambda: native.qkv_split(qkv, cos, sin, Hq, Hkv)),
        ("qkv_merge_rope", 2 * qkv.numel() * e2, lambda: native.qkv_merge(q, k, v, cos, sin)),
        ("cross_entropy", logits.numel() * e2, lambda: native.cross_entropy(logits, labels)),
        ("cross_entropy_bwd", 2 * logits.numel() * e2, lambda: native.cross_entropy_bwd(dloss, logits, labels, lse)),
        ("embedding", 2 * n * e2, lambda: native.embedding(ids, table)),
        ("embedding_bwd", n * e2 + V * H * (4 + 4 + e2), lambda: native.embedding_bwd(dy, ids, V)),
        ("colsum", n * e2, lambda: native.colsum(dy)),
        ("dropout", 2 * n * e2, lambda: native.dropout(x, 0.1, seed, 7)),
        ("adamw", n * (4 * 4 + 3 * 4 + 2), lambda: native.adamw(pm, pg, m_, v_, step, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1.0, bf, None, False)),
        ("router", rl.numel() * 4 * 2 + rl.shape[0] * 2 * 12, lambda: torch.ops.b200moe.router(rl, 2)),
    ]
    for name, nbytes, fn in cases:
        ms = timed(fn, iters, warmup, flush)
        print(json.dumps({"op": name, "rows": R, "hidden": H, "algorithmic_mb": round(nbytes / 1e6, 1), "ms": round(ms, 4),
                          "gbs": round(nbytes / ms / 1e6, 1), "frac_of_measured_copy_bw": round(nbytes / ms / 1e6 / bw_peak, 3),
                          "status": native.read_status()}), flush=True)


_KEEP = contextlib.ExitStack()   # flag overrides that last until the process ends


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "gemm_batched", "attn_fwd", "attn_bwd", "rmsnorm", "rmsnorm_bwd", "swiglu", "cross_entropy",
                                   "adamw", "suite"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", default="fwd", choices=["fwd", "dgrad", "wgrad"])
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--experts", type=int, default=4)
    ap.add_argument("--fill", type=float, default=1.0,
                    help="gemm_batched: fraction of each group's rows that hold data (< 1: the unequal-group kernel, which "
                         "skips the rest; the FLOP count stays that of the full storage, so the rate reads as 'effective')")
    a = ap.parse_args()
    native.load()
    if a.op == "suite":
        return suite(a.rows, a.hidden, a.iters, a.warmup, not a.no_flush)
    tf_peak, bw_peak = _peaks()
    bf = torch.bfloat16
    rnd = lambda *s: torch.randn(*s, device="cuda", dtype=bf)
    flops = bytes_ = 0
    fn_equal = None   # gemm_batched --fill: the same data through the equal-group kernel, timed in the same process
    if a.op == "gemm":
        M, N, K = a.m, a.n, a.k
        flops = 2.0 * M * N * K
        if a.layout == "fwd":
            x, w = rnd(M, K), rnd(N, K)
            fn = lambda: native.linear(x, w, None)
        elif a.layout == "dgrad":
            dy, w = rnd(M, N), rnd(N, K)
            fn = lambda: native.linear_dgrad(dy, w)
        else:
            dy, x = rnd(M, N), rnd(M, K)
            fn = lambda: native.linear_wgrad(dy, x)
    elif a.op == "gemm_batched":
        E, M, N, K = a.experts, a.m, a.n, a.k
        flops = 2.0 * E * M * N * K
        xb, wb = rnd(E, M, K), rnd(E, N, K)
        if a.fill < 1.0:
            from ..utils import config

            _KEEP.enter_context(config.moe_skip_empty_slots.set(2))   # row counts used by all three GEMMs
            live = int(M * a.fill)
            xb[:, live:] = 0
            counts = torch.full((E, 1), live, dtype=torch.int32, device="cuda")
            dyb = rnd(E, M, N)
            dyb[:, live:] = 0
            if a.layout == "fwd":
                fn, fn_equal = (lambda: native.linear_batched(xb, wb, counts, M)), (lambda: native.linear_batched(xb, wb))
            elif a.layout == "dgrad":
                fn, fn_equal = (lambda: native.linear_dgrad_batched(dyb, wb, counts, M)), (lambda: native.linear_dgrad_batched(dyb, wb))
            else:
                fn = lambda: native.linear_wgrad_batched(dyb, xb, torch.float32, counts, M)
                fn_equal = lambda: native.linear_wgrad_batched(dyb, xb, torch.float32)
        else:
            fn = lambda: native.linear_batched(xb, wb)
    elif a.op in ("attn_fwd", "attn_bwd"):
        B, S, H, D = a.batch, a.seq, a.heads, a.head_dim
        Hkv = a.kv_heads or H
        q, k, v, do = rnd(B, S, H, D), rnd(B, S, Hkv, D), rnd(B, S, Hkv, D), rnd(B, S, H, D)
        scale = D ** -0.5
        o, lse = att.attention_fwd(q, k, v, True, scale)
        fwd_flops = 4.0 * B * H * S * S * D / 2
        if a.op == "attn_fwd":
            flops, fn = fwd_flops, (lambda: att.attention_fwd(q, k, v, True, scale))
        else:
            flops, fn = 2.5 * fwd_flops, (lambda: att.attention_bwd(do, q, k, v, o, lse, True, scale))
    elif a.op in ("rmsnorm", "rmsnorm_bwd"):
        x, w, dy = rnd(a.rows, a.hidden), rnd(a.hidden), rnd(a.rows, a.hidden)
        _, rstd = native.rmsnorm(x, w, 1e-5)
        if a.op == "rmsnorm":
            bytes_, fn = 2.0 * x.numel() * 2, (lambda: native.rmsnorm(x, w, 1e-5))
        else:
            bytes_, fn = 3.0 * x.numel() * 2, (lambda: native.rmsnorm_bwd(dy, x, w, rstd))
    elif a.op == "swiglu":
        gu = rnd(a.rows, 2 * a.hidden)
        bytes_, fn = 3.0 * a.rows * a.hidden * 2, (lambda: native.swiglu(gu))
    elif a.op == "cross_entropy":
        logits = rnd(a.rows, a.hidden)
        labels = torch.randint(0, a.hidden, (a.rows,), device="cuda")
        bytes_, fn = 1.0 * logits.numel() * 2, (lambda: native.cross_entropy(logits, labels))
    else:  # adamw
        n = a.rows * a.hidden
        p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        step = torch.ones((), dtype=torch.int64, device="cuda")
        bytes_ = n * (4 * 4 + 3 * 4 + 2)
        fn = lambda: native.adamw(p, g, m, v, step, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1.0, bf, None, False)
    ms = timed(fn, a.iters, a.warmup, not a.no_flush)
    torch.cuda.synchronize()
    out = {"op": a.op, "ms": round(ms, 4), "status": native.read_status()}
    if fn_equal is not None:
        out["fill"] = a.fill
        out["ms_equal_groups_same_data"] = round(timed(fn_equal, a.iters, a.warmup, not a.no_flush), 4)
        out["ms_again"] = round(timed(fn, a.iters, a.warmup, not a.no_flush), 4)
    out.update({k: v for k, v in vars(a).items() if k in ("m", "n", "k", "layout", "batch", "seq", "heads", "head_dim", "rows", "hidden")})
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_measured_burst_peak"] = round(flops / ms / 1e9 / tf_peak, 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        out["frac_of_measured_copy_bw"] = round(bytes_ / ms / 1e6 / bw_peak, 3)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
