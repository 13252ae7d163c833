"""Pipelined training of a small decoder-block model, validated against the same step run without pipelining.

    python examples/basic.py --pp 2                      # both pipeline ranks in this process (single controller)
    python examples/basic.py --pp 2 --multi-process      # one process per pipeline rank (gloo on CPU, NCCL on GPUs)
    python examples/basic.py --pp 4 --schedule interleaved --num-ubatches 8 --device cuda

Every stage holds two blocks (attention + GELU MLP, post-LayerNorm); the loss is the mean squared error against
the input; the optimizer is Adam on fp32 master weights (the compute copy is fp32 on CPU, bf16 on GPUs, where the
ops are the native sm_100a kernels; ``--dtype float32 --device cuda`` runs the same ops through their torch forms).  The first step's gradients, parameters, losses and predictions are compared
with the un-pipelined run, then both are trained side by side and their losses compared at every step.  This is
the counterpart of the reference's examples/basic.py:93-345 on this framework's API.
"""
from __future__ import annotations

import argparse
import os
import sys
from contextlib import contextmanager

import torch
from torch.utils import _pytree as pytree

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import jaxpp_b200 as jp  # noqa: E402
from jaxpp_b200.ops import core as ops  # noqa: E402

HIDDEN, HEADS, FFN, BATCH, SEQ = 64, 4, 192, 4, 32        # CPU sizes; ``use_gpu_sizes`` switches to head_dim 64


def use_gpu_sizes():
    """The flash-attention kernels take head dimensions 64 and 128."""
    global HIDDEN, HEADS, FFN, BATCH, SEQ
    HIDDEN, HEADS, FFN, BATCH, SEQ = 256, 4, 768, 4, 128


def init_params(n_blocks: int, dtype, device, seed: int = 0) -> list:
    g = torch.Generator().manual_seed(seed)
    w = lambda *s: (torch.randn(*s, generator=g) * 0.08).to(dtype).to(device)
    zeros = lambda n: torch.zeros(n, dtype=dtype, device=device)
    ones = lambda n: torch.ones(n, dtype=dtype, device=device)
    return [{"wqkv": w(3 * HIDDEN, HIDDEN), "wo": w(HIDDEN, HIDDEN), "w1": w(FFN, HIDDEN), "b1": zeros(FFN),
             "w2": w(HIDDEN, FFN), "g1": ones(HIDDEN), "be1": zeros(HIDDEN), "g2": ones(HIDDEN), "be2": zeros(HIDDEN)}
            for _ in range(n_blocks)]


def block(p: dict, x: torch.Tensor) -> torch.Tensor:
    b, s, h = x.shape
    flat = x.reshape(b * s, h)
    qkv = ops.linear(flat, p["wqkv"], None).view(b, s, 3, HEADS, h // HEADS)
    q, k, v = (qkv[:, :, i].transpose(1, 2).contiguous() for i in range(3))          # [b, heads, s, hd]
    att = ops.attention(q, k, v, False, (h // HEADS) ** -0.5)[0].transpose(1, 2).reshape(b * s, h)
    flat = ops.layernorm(flat + ops.linear(att, p["wo"], None), p["g1"], p["be1"], 1e-5)[0]
    mlp = ops.linear(ops.gelu(ops.linear(flat, p["w1"], p["b1"])), p["w2"], None)
    return ops.layernorm(flat + mlp, p["g2"], p["be2"], 1e-5)[0].view(b, s, h)


def forward(params: list, x: torch.Tensor, n_stages: int) -> torch.Tensor:
    per_stage = len(params) // n_stages
    for i, p in enumerate(params):
        x = block(p, x)
        if (i + 1) % per_stage == 0:
            x = jp.mark_stage_end(x)       # everything since the previous marker is one pipeline stage
    return x


def make_step(schedule, n_ubatches: int, lr: float):
    """``(params, master, m, v, count, batch[n_ubatches, ...]) -> (params', master', m', v', count', losses,
    predictions)``; ``params`` is the compute copy, ``master`` / ``m`` / ``v`` are fp32."""

    def step(params, master, m, v, count, batch):
        def microbatch(mb):
            def loss_fn(p):
                out = forward(p, mb, schedule.num_stages)
                return ((out - mb) ** 2).mean() / n_ubatches, out

            (loss, pred), grads = jp.value_and_grad(loss_fn, has_aux=True)(params)
            return (loss, pred), grads

        # losses / predictions are stacked over microbatches (Concat), gradients summed (Add)
        (losses, preds), grads = jp.treduce(microbatch, batch, schedule=schedule)
        new_count = count + 1
        upd = pytree.tree_map(   # fused AdamW: new master, moments and the low-precision copy in one kernel
            lambda p, ma, g, mm, vv: ops.adamw(ma, g, mm, vv, new_count, lr, 0.9, 0.999, 1e-8, 0.0, 1.0, p.dtype),
            params, master, grads, m, v)
        pick = lambda k: pytree.tree_map(lambda p, u: u[k], params, upd, is_leaf=lambda x: isinstance(x, tuple))
        return pick(3), pick(0), pick(1), pick(2), new_count, losses, preds

    return step


@contextmanager
def checking(name: str, verbose: bool):
    if verbose:
        print(f"[*] `{name}` validation {'.' * (60 - len(name))} ", end="", flush=True)
    try:
        yield
    except AssertionError:
        if verbose:
            print("FAIL")
        raise
    if verbose:
        print("PASS")


def local(x):
    """The tensor this process holds of a result (None when it lives on another pipeline rank only)."""
    return x.local_tensor() if isinstance(x, jp.MpmdArray) else x


def compare(ref, got, rtol, atol):
    a = pytree.tree_leaves(ref)
    b = pytree.tree_leaves(got, is_leaf=lambda x: isinstance(x, jp.MpmdArray))
    assert len(a) == len(b)
    for x, y in zip(a, b):
        t = local(y)
        if t is not None:
            torch.testing.assert_close(t.float().cpu(), x.float().cpu(), rtol=rtol, atol=atol)


def make_schedule(name: str, pp: int):
    if name == "std":
        return jp.Std1F1B(pp)
    if name == "eager":
        return jp.Eager1F1B(pp)
    if name == "gpipe":
        return jp.GPipe(pp)
    if name == "zb":
        return jp.ZeroBubble(pp)
    if name == "interleaved":
        return jp.Interleaved1F1B(2 * pp, pp)
    if name == "dualpipev":
        return jp.DualPipeV(2 * pp, pp)
    raise SystemExit(f"unknown schedule {name}")


def run(args):
    import torch.distributed as dist

    multi = dist.is_available() and dist.is_initialized()
    kind = args.device
    mesh = jp.MpmdMesh.create({"mpmd": args.pp, "data": 1, "model": 1}, kind=kind, multi_process=multi)
    device = mesh.my_device.torch_device if multi else torch.device(kind)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype or ("bfloat16" if kind == "cuda" else "float32")]
    verbose = not multi or dist.get_rank() == 0
    if kind == "cuda":
        use_gpu_sizes()
        if dtype == torch.float32:   # the native kernels are bf16: run the ops through their torch forms instead
            from jaxpp_b200.utils import config

            config.use_native_kernels.set(False).__enter__()
    schedule = make_schedule(args.schedule, args.pp)
    params = init_params(2 * schedule.num_stages, dtype, device)
    zeros = lambda: pytree.tree_map(lambda p: torch.zeros_like(p, dtype=torch.float32), params)
    master = lambda: pytree.tree_map(lambda p: p.float().clone(), params)
    count = torch.zeros((), dtype=torch.int64, device=device)
    batch = torch.rand(args.num_ubatches, BATCH, SEQ, HIDDEN, generator=torch.Generator().manual_seed(1)).to(dtype).to(device)

    step = make_step(schedule, args.num_ubatches, 0.005)
    pipelined = jp.mpmd_jit_with_loop(step, mesh)       # called like `step`; returns MpmdArrays

    ref = step(params, master(), zeros(), zeros(), count, batch)  # eager call = the sequential oracle
    got = pipelined(params, master(), zeros(), zeros(), count, batch)
    if local(got[5]) is not None:     # the losses live on the rank of the last stage
        print(f"first step, pipelined loss per microbatch: {local(got[5]).float().cpu().numpy()}", flush=True)
    if verbose:
        print(f"\n{'=' * 30} VALIDATION {'=' * 30}\n")
    exact = dtype == torch.float32 and kind == "cpu"
    rtol = atol = 0.0 if exact else (1e-3 if dtype == torch.float32 else 2e-2)
    for name, idx in (("optimizer state", (1, 2, 3, 4)), ("params", (0,)), ("loss", (5,)), ("prediction", (6,))):
        with checking(name, verbose):
            compare([ref[i] for i in idx], [got[i] for i in idx], rtol, atol)

    if verbose:
        print(f"\n{'=' * 26} TRAINING: {args.train_steps:04d} steps {'=' * 26}")
    for i in range(args.train_steps):
        ref = step(*ref[:5], batch)
        got = pipelined(*got[:5], batch)                # MpmdArrays go straight back in
        compare(ref[5], got[5], rtol, max(atol, 1e-4))
        mine = local(got[5])
        if mine is not None and (i == 0 or (i + 1) % 10 == 0):
            print(f"[{i + 1:04d}/{args.train_steps:04d}] loss {float(ref[5].float().sum()):.6f} (sequential) "
                  f"{float(mine.float().sum()):.6f} (pipelined)")
    if verbose:
        print("\nSUCCESS")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--pp", type=int, default=2, help="pipeline ranks")
    ap.add_argument("--num-ubatches", "--num_ubatches", type=int, default=8, help="microbatches per step")
    ap.add_argument("--train-steps", "--train_steps", type=int, default=20)
    ap.add_argument("--dtype", choices=["float32", "bfloat16"], default=None, help="default: float32 on CPU, bfloat16 on GPUs")
    ap.add_argument("--schedule", default="std", choices=["std", "eager", "gpipe", "zb", "interleaved", "dualpipev"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu", choices=["cpu", "cuda"])
    ap.add_argument("--multi-process", action="store_true", help="one process per pipeline rank")
    ap.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.worker:
        from jaxpp_b200.launch import distributed_main

        distributed_main(lambda: run(args), backend="gloo" if args.device == "cpu" else "nccl")
    elif args.multi_process and args.pp > 1:
        from jaxpp_b200.launch import launch

        env = {"CUDA_VISIBLE_DEVICES": ""} if args.device == "cpu" else {}
        rest = [a for a in (sys.argv[1:] if argv is None else argv) if a != "--multi-process"]
        sys.exit(launch([os.path.abspath(__file__), "--worker", *rest], args.pp, env=env, timeout_s=1800))
    else:
        run(args)


if __name__ == "__main__":
    main()
