"""Per-op timings of the fused tensor-parallel kernels against their NCCL twins (collective kernel + GEMM).

Run one process per GPU::

    python -m jaxpp_b200.launch --nproc 2 -m jaxpp_b200.parallel.microbench [--d-model 4096 --ffn 11008 --tokens 16384]

Shapes default to one Llama-2-7B layer under TP = number of ranks with sequence parallelism: the five ops the
forward and backward of a column- / row-parallel linear pair launch.  Every number is device time (CUDA
events), max over ranks, after warm-up, with a 256 MiB write between iterations to flush L2.  The target of the
roofline column is max(FLOPs / GEMM peak, bytes crossing NVLink per rank / link bandwidth).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

PEAK_TFLOPS = 1677.8     # measured cuBLAS bf16 burst on this hardware
LINK_GBS = 770.0         # measured peer copy, one direction


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f).get("bf16_tflops", PEAK_TFLOPS))
    except Exception:
        return PEAK_TFLOPS


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)
        dist.barrier()
        # keep the GPU busy for ~0.5 ms while the host prepares the launch (descriptor set-up, tensor maps), so that
        # the events bracket device time only, as they do inside a training step where the host runs ahead
        torch.cuda._sleep(1_000_000)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per microbatch over the whole TP group")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import jaxpp_b200 as jp
    from jaxpp_b200.launch import distributed_main
    from jaxpp_b200.ops import core as ops
    from jaxpp_b200.ops import native
    from jaxpp_b200.parallel import fused
    from jaxpp_b200.utils import config

    def body():
        n, r = dist.get_world_size(), dist.get_rank()
        peak = _peaks()
        mesh = jp.MpmdMesh.create({"mpmd": 1, "data": 1, "model": n}, kind="cuda", multi_process=True)
        T, D, F = args.tokens, args.d_model, args.ffn
        Tl = T // n
        flush = torch.zeros(64 << 20, device="cuda")
        g = torch.Generator(device="cuda").manual_seed(r)
        rnd = lambda *s: (torch.randn(*s, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
        x_shard, dy_shard = rnd(Tl, D), rnd(Tl, D)
        rows = []
        with mesh:
            cases = []
            for name, nout in (("qkv", 3 * D // n), ("gate_up", 2 * (F // n))):
                w = rnd(nout, D)
                dy = rnd(T, nout)
                cases.append((f"ag_linear[{name}]", lambda w=w: torch.ops.b200tp.ag_linear(x_shard, w, None, "model"),
                              2.0 * T * nout * D, (n - 1) * Tl * D * 2))
                cases.append((f"dgrad_rs[{name}]", lambda w=w, dy=dy: torch.ops.b200tp.dgrad_rs(dy, w, "model"),
                              2.0 * T * nout * D, (n - 1) * Tl * D * 2))
                cases.append((f"ag_wgrad[{name}]", lambda dy=dy: torch.ops.b200tp.ag_wgrad(dy, x_shard, "model", torch.float32),
                              2.0 * T * nout * D, (n - 1) * Tl * D * 2))
            for name, kin in (("wo", D // n), ("down", F // n)):
                w = rnd(D, kin)
                x = rnd(T, kin)
                cases.append((f"linear_rs[{name}]", lambda w=w, x=x: torch.ops.b200tp.linear_rs(x, w, "model"),
                              2.0 * T * D * kin, (n - 1) * Tl * D * 2))
                cases.append((f"ag_dgrad[{name}]", lambda w=w: torch.ops.b200tp.ag_dgrad(dy_shard, w, "model"),
                              2.0 * T * D * kin, (n - 1) * Tl * D * 2))
            for name, fn, flops, link_bytes in cases:
                t_fused = _time(fn, args.iters, flush)
                with config.use_fused_collectives.set(False):
                    t_nccl = _time(fn, args.iters, flush)
                target = max(flops / (peak * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3
                rows.append(dict(op=name, fused_ms=round(t_fused, 4), nccl_ms=round(t_nccl, 4),
                                 speedup=round(t_nccl / t_fused, 3), tflops=round(flops / t_fused / 1e9, 1),
                                 target_ms=round(target, 4), of_target=round(target / t_fused, 3)))
            # plain GEMM of the same local shape, for reference
            w = rnd(3 * D // n, D)
            xf = rnd(T, D)
            t_plain = _time(lambda: ops.linear(xf, w, None), args.iters, flush)
            torch.cuda.synchronize()
            status = native.read_status()
        if r == 0:
            out = dict(n_ranks=n, tokens=T, d_model=D, ffn=F, peak_tflops_of_measured=peak, link_gbs=LINK_GBS,
                       plain_gemm_qkv_ms=round(t_plain, 4), kernel_status=status, fallbacks=fused.FALLBACKS[0], ops=rows)
            text = json.dumps(out, indent=1)
            print(text, flush=True)
            if args.out:
                with open(args.out, "w") as f:
                    f.write(text + "\n")

    distributed_main(body)


if __name__ == "__main__":
    main()
