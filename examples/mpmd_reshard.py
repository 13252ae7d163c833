"""Moving arrays between an SPMD layout over the whole mesh and the MPMD (per pipeline rank) layout.

    python examples/mpmd_reshard.py                      # 2 pipeline ranks of one CPU device each, in one process
    python examples/mpmd_reshard.py --multi-process      # 2 stages x 2 "fsdp" ranks, one process per device

Weights are created sharded over *all* devices (the stage axis included, which is the memory-efficient way to
initialise or to load a checkpoint), the accumulation loop is compiled, ``compiled.in_shardings`` says which
pipeline rank needs which argument, ``spmd_to_mpmd_reshard`` moves every array to its rank (the sources are
deleted), the loop runs, and ``mpmd_to_spmd_reshard`` spreads the gradients back over the whole mesh.
Sharding inside a pipeline rank is explicit in this framework: the weights are whole on every device of their
rank, the batch is split over the ``fsdp`` axis, and the step sums the gradients over that axis itself.
Counterpart of the reference's examples/mpmd_reshard.py:33-139.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import jaxpp_b200 as jp  # noqa: E402
from jaxpp_b200.array import DistArray  # noqa: E402
from jaxpp_b200.ops import core as ops  # noqa: E402
from jaxpp_b200.parallel import tp  # noqa: E402

P = jp.PartitionSpec
EMBED, HIDDEN = 64, 256


def run(args):
    import torch.distributed as dist

    multi = dist.is_available() and dist.is_initialized()
    say = (lambda *a: print(f"[{dist.get_rank()}]", *a, flush=True)) if multi else print
    fsdp = 2 if multi else 1     # one process drives pipeline ranks of a single device each
    mesh = jp.MpmdMesh.create({"stage": 2, "fsdp": fsdp, "tensor": 1}, kind=args.device, multi_process=multi,
                              mpmd_axis_name="stage")
    whole = mesh.jax_mesh                                        # every device, stage axis included

    specs = [P(("stage", "fsdp"), "tensor"), P("tensor", ("stage", "fsdp")), P("fsdp", None, None)]
    shardings = [jp.NamedSharding(whole, s) for s in specs]
    g = torch.Generator().manual_seed(0)
    dtype = torch.float32 if args.device == "cpu" else torch.bfloat16      # the native GEMM kernels are bf16
    full = [(torch.randn(HIDDEN, EMBED, generator=g) * 0.05).to(dtype), (torch.randn(EMBED, HIDDEN, generator=g) * 0.05).to(dtype),
            torch.randn(4, 32, EMBED, generator=g).to(dtype)]
    # SPMD initialisation: every process keeps only the shards of its own devices
    mine = [mesh.my_device] if multi else None
    W1, W2, x = (DistArray.from_global(t, s, devices=mine) for t, s in zip(full, shardings))

    def grads_of_microbatch(weights, xb):
        def loss(ws):
            w1, w2 = ws
            flat = xb.reshape(-1, EMBED)
            h1 = jp.pipeline_enter_stage(ops.linear(flat, w1, None))
            h2 = jp.pipeline_enter_stage(ops.linear(h1, w2, None))
            return ((flat - h2) ** 2).sum()

        return jp.value_and_grad(loss)(weights)[1]

    def accumulation_loop(W1, W2, x, unused):
        g1, g2 = jp.treduce(lambda xb: grads_of_microbatch((W1, W2), xb), x, schedule=jp.Std1F1B(mesh.mpmd_dim),
                            operation=jp.Add)
        if fsdp > 1:   # every fsdp rank saw its own slice of each microbatch
            g1, g2 = tp.all_reduce(g1, "fsdp"), tp.all_reduce(g2, "fsdp")
        return g1, g2

    # layout inside a pipeline rank: weights whole, every microbatch split over the fsdp axis
    mb_spec = P(None, "fsdp", None)
    loop = jp.mpmd_jit_with_loop(accumulation_loop, mesh, in_specs=(P(), P(), mb_spec, mb_spec), out_specs=(P(), P()))
    like = lambda t, split=1: jp.ShapeDtypeStruct((t.shape[0], t.shape[1] // split, *t.shape[2:]), t.dtype)
    compiled = loop.compile(like(full[0]), like(full[1]), like(full[2], fsdp), like(full[2], fsdp))
    arg_shardings, _ = compiled.in_shardings
    for name, s in zip(("W1", "W2", "x", "unused"), arg_shardings):
        say(f"{name}: needed on pipeline ranks {sorted(s.mesh_ids)} with spec {s.spec}")

    unused = DistArray.from_global(full[2], shardings[2], devices=mine)
    _W1, _W2, _x, _unused = jp.spmd_to_mpmd_reshard(mesh, [W1, W2, x, unused], list(arg_shardings))
    say(f"sources deleted: {W1.is_deleted()=} {W2.is_deleted()=} {x.is_deleted()=}")
    W1, W2, x = _W1, _W2, _x
    say(f"W1 on ranks {W1.mpmd_idxs}, addressable here: {W1.is_partially_addressable}")
    say(f"W2 on ranks {W2.mpmd_idxs}, addressable here: {W2.is_partially_addressable}")

    dW1, dW2 = compiled(W1, W2, x, _unused)
    dW1, dW2 = jp.mpmd_to_spmd_reshard(mesh, [dW1, dW2], shardings[:2])
    say(f"dW1 sharding: {dW1.sharding.spec}; dW2 sharding: {dW2.sharding.spec}")

    # check against plain autograd on the full arrays
    w1, w2 = full[0].float().requires_grad_(), full[1].float().requires_grad_()
    flat = full[2].float().reshape(-1, EMBED)
    ((flat - (flat @ w1.T) @ w2.T) ** 2).sum().backward()
    tol = 1e-4 if dtype == torch.float32 else 5e-2
    for got, want, name in ((dW1, w1.grad, "dW1"), (dW2, w2.grad, "dW2")):
        for dev, shard in got.shards.items():
            idx = got.sharding.device_index(dev, want.shape)
            torch.testing.assert_close(shard.float().cpu(), want[idx], rtol=tol, atol=tol * float(want.abs().max()))
    say("gradients match plain autograd")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--multi-process", action="store_true")
    ap.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.worker:
        from jaxpp_b200.launch import distributed_main

        distributed_main(lambda: run(args), backend="gloo" if args.device == "cpu" else "nccl")
    elif args.multi_process:
        from jaxpp_b200.launch import launch

        env = {"CUDA_VISIBLE_DEVICES": ""} if args.device == "cpu" else {}
        sys.exit(launch([os.path.abspath(__file__), "--worker", "--device", args.device], 4, env=env, timeout_s=600))
    else:
        run(args)


if __name__ == "__main__":
    main()
