"""Forward-only pipelining with ``mpmd_jit_by_yield``: no microbatch loop, the stages of one forward pass are
placed round-robin on the pipeline ranks (stage ``s`` on rank ``s % pp``) and run in order, with the activation
handed from rank to rank.

    python examples/inference.py --pp 2 --stages 4
    python examples/inference.py --pp 2 --stages 4 --multi-process

A small Llama-style language model scores a batch of token sequences; the per-sequence log-likelihood is compared
with the un-pipelined forward.  Counterpart of the reference's forward-only entry point (core.py:3120-3148, 3926).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import jaxpp_b200 as jp  # noqa: E402
from jaxpp_b200.models import transformer as tf  # noqa: E402
from jaxpp_b200.ops import core as ops  # noqa: E402


def run(args):
    import torch.distributed as dist

    multi = dist.is_available() and dist.is_initialized()
    mesh = jp.MpmdMesh.create({"mpmd": args.pp, "data": 1, "model": 1}, kind=args.device, multi_process=multi)
    device = mesh.my_device.torch_device if multi else torch.device(args.device)
    dtype = torch.float32 if args.device == "cpu" else torch.bfloat16
    # head_dim 64: one of the sizes the flash-attention kernels take
    cfg = tf.ModelConfig("llama", vocab=512, d_model=256, n_layers=args.stages * 2, n_heads=4, n_kv_heads=2, ffn=512, seq=128,
                         n_stages=args.stages, dtype=dtype)
    params = tf.init_params(cfg, device, seed=0)
    rope = tf.rope_tables(cfg, device)
    g = torch.Generator().manual_seed(2)
    tokens = torch.randint(0, cfg.vocab, (4, cfg.seq + 1), generator=g).to(device)

    def score(params, tokens):
        """log p(tokens[:, 1:] | tokens[:, :-1]) per sequence"""
        inp, nxt = tokens[:, :-1], tokens[:, 1:]
        x = ops.embedding(inp.reshape(-1), params["embed"])
        x = tf.run_layers(cfg, params, x, inp.shape[0], rope)          # marks the end of every stage but the last
        x = ops.rmsnorm(x, params["final_norm"], cfg.eps)[0]
        nll, _ = ops.cross_entropy(ops.linear(x, params["lm_head"], None), nxt.reshape(-1))
        return jp.mark_stage_end(-nll.view(inp.shape[0], -1).sum(-1))

    want = score(params, tokens)
    pipelined = jp.mpmd_jit_by_yield(score, mesh)
    got = pipelined(params, tokens)
    mine = got.local_tensor()
    if mine is not None:       # the result lives on the rank of the last stage
        tol = 0.0 if args.device == "cpu" else 5e-2
        torch.testing.assert_close(mine.float().cpu(), want.float().cpu(), rtol=tol, atol=tol)
        print(f"log-likelihood per sequence (pipelined over {args.pp} ranks, {args.stages} stages): "
              f"{[round(float(v), 3) for v in mine.float().cpu()]} -- matches the un-pipelined forward", flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--stages", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu", choices=["cpu", "cuda"])
    ap.add_argument("--multi-process", action="store_true")
    ap.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.worker:
        from jaxpp_b200.launch import distributed_main

        distributed_main(lambda: run(args), backend="gloo" if args.device == "cpu" else "nccl")
    elif args.multi_process and args.pp > 1:
        from jaxpp_b200.launch import launch

        env = {"CUDA_VISIBLE_DEVICES": ""} if args.device == "cpu" else {}
        rest = [a for a in (sys.argv[1:] if argv is None else argv) if a != "--multi-process"]
        sys.exit(launch([os.path.abspath(__file__), "--worker", *rest], args.pp, env=env, timeout_s=600))
    else:
        run(args)


if __name__ == "__main__":
    main()
