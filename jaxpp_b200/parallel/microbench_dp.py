"""Timings of the data-parallel collectives over peer memory against NCCL: all-reduce, reduce-scatter and
all-gather of gradient- / parameter-sized flat tensors.

Run one process per GPU::

    python -m jaxpp_b200.launch --nproc 2 -m jaxpp_b200.parallel.microbench_dp [--mib 64 256 1024]

Every number is device time (CUDA events), max over ranks, after warm-up, with a 256 MiB write between
iterations to flush L2.  Bus bandwidth follows the usual convention: all-reduce 2 (n-1)/n * bytes / t,
reduce-scatter and all-gather (n-1)/n * bytes / t, with ``bytes`` the size of the full tensor; the link
denominator is the measured peer copy bandwidth of one direction.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

LINK_GBS = 770.0         # measured peer copy, one direction


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)
        dist.barrier()
        torch.cuda._sleep(1_000_000)   # the host prepares the launch while the GPU is busy: events bracket device time
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
    ap.add_argument("--mib", type=int, nargs="+", default=[64, 256, 1024], help="sizes of the full fp32 tensor")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import jaxpp_b200 as jp
    from jaxpp_b200.launch import distributed_main
    from jaxpp_b200.ops import native
    from jaxpp_b200.parallel import fused, zero

    def body():
        n, r = dist.get_world_size(), dist.get_rank()
        mesh = jp.MpmdMesh.create({"mpmd": 1, "data": n, "model": 1}, kind="cuda", multi_process=True)
        flush = torch.zeros(64 << 20, device="cuda")
        rows = []
        with mesh:
            for mib in args.mib:
                numel = mib * (1 << 20) // 4
                g = torch.randn(numel, device="cuda")
                s = zero.shard_numel(numel, n)
                shard_bf16 = torch.randn(s, device="cuda").to(torch.bfloat16)
                padded = torch.zeros(s * n, device="cuda")
                rs_out, ag_out = torch.empty(s, device="cuda"), torch.empty(s * n, dtype=torch.bfloat16, device="cuda")

                def nccl_ar():
                    t = g.clone()
                    dist.all_reduce(t)

                def nccl_rs():
                    padded[:numel].copy_(g)
                    dist.reduce_scatter_tensor(rs_out, padded)

                cases = [
                    ("all_reduce fp32", lambda: fused.all_reduce(g, "data"), nccl_ar, 2.0 * (n - 1) / n * numel * 4),
                    ("reduce_scatter fp32", lambda: fused.reduce_scatter_flat(g, "data"), nccl_rs, (n - 1) / n * numel * 4),
                    ("all_gather bf16", lambda: fused.all_gather_flat(shard_bf16, "data"),
                     lambda: dist.all_gather_into_tensor(ag_out, shard_bf16), (n - 1) / n * s * n * 2),
                ]
                for name, f_fused, f_nccl, bus_bytes in cases:
                    t_f, t_n = _time(f_fused, args.iters, flush), _time(f_nccl, args.iters, flush)
                    rows.append(dict(op=name, mib=mib, fused_ms=round(t_f, 4), nccl_ms=round(t_n, 4),
                                     speedup=round(t_n / t_f, 3), fused_bus_gbs=round(bus_bytes / t_f / 1e6, 1),
                                     of_link=round(bus_bytes / t_f / 1e6 / LINK_GBS, 3)))
            torch.cuda.synchronize()
            status = native.read_status()
        if r == 0:
            text = json.dumps(dict(n_ranks=n, link_gbs=LINK_GBS, kernel_status=status, ops=rows), indent=1)
            print(text, flush=True)
            if args.out:
                with open(args.out, "w") as f:
                    f.write(text + "\n")

    distributed_main(body)


if __name__ == "__main__":
    main()
