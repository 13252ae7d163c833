"""Training driver: run any named configuration with checkpoint/resume, failure detection and step metrics.

    python -m jaxpp_b200.launch --nproc 8 -m ...            (or torch.distributed.run)
    python -m jaxpp_b200.train --config llama7b_pp4tp2 --steps 100 --ckpt-dir /data/ckpt --ckpt-every 50 --metrics m.jsonl

One process per device; ``--device cpu`` with ``--tiny`` runs the same program structure at toy sizes over gloo
(what the tests do).  On resume the latest complete checkpoint under ``--ckpt-dir`` is loaded into this run's
layout, the data cursor and step counter continue from it.
"""
from __future__ import annotations

import argparse
import dataclasses

import torch


def main(argv=None):
    import jaxpp_b200 as jp
    from jaxpp_b200 import checkpoint as ckpt
    from jaxpp_b200 import configs, fault
    from jaxpp_b200.launch import distributed_main
    from jaxpp_b200.metrics import StepMetrics
    from jaxpp_b200.models import lm_trainer as lt

    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--device", default=None, choices=[None, "cpu", "cuda"])
    ap.add_argument("--tiny", action="store_true", help="shrink the model (same structure) for smoke runs")
    ap.add_argument("--ckpt-dir", default=None)
    ap.add_argument("--ckpt-every", type=int, default=0)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--metrics", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--clip-grad-norm", type=float, default=None, help="clip gradients to this global L2 norm")
    ap.add_argument("--stage-layers", default="equal",
                    help="blocks per pipeline stage: 'equal', 'auto' (even out the pipeline ranks' work) or a list such as "
                         "4,4,4,4,4,4,4.5,3.5 (a stage may end between the attention half and the feed-forward half of a block)")
    ap.add_argument("--shard-optimizer", action="store_true",
                    help="keep master weights and Adam moments as 1/dp slices per data-parallel rank (ZeRO stage 1)")
    args = ap.parse_args(argv)

    def run():
        import torch.distributed as dist

        rc = configs.get(args.config)
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        if world not in (1, rc.n_gpus):
            raise SystemExit(f"{rc.name} needs {rc.n_gpus} processes, got {world}")
        kind = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
        over = {}
        if args.tiny:
            over = dict(vocab=256, d_model=64, n_layers=rc.n_stages * 1, n_heads=4, n_kv_heads=2 if rc.model().n_kv_heads != rc.model().n_heads else 4,
                        ffn=128, seq=32, dtype=torch.float32 if kind == "cpu" else torch.bfloat16)
            if rc.ep > 1:
                over.update(n_experts=2 * rc.ep, capacity_factor=4.0)
        cfg = dataclasses.replace(rc.model_config(), **over) if over else rc.model_config()
        if cfg.family == "encoder":
            raise SystemExit("the encoder configuration is exercised by tests/test_models.py; train.py drives language models")
        multi = world > 1
        mesh = jp.MpmdMesh.create(rc.mesh_shape() if multi else {"mpmd": rc.pp, "data": 1, "model": 1}, kind=kind, multi_process=multi)
        if not multi and (rc.tp > 1 or rc.dp > 1):
            raise SystemExit("tensor/data parallel configurations need one process per device")
        sched = rc.make_schedule()
        sizes = configs.choose_stage_layers(cfg, sched, rc.pp, max(1, rc.microbatch // rc.dp) * cfg.seq, args.stage_layers)
        if sizes is not None:
            cfg = dataclasses.replace(cfg, stage_layers=sizes)
        device = mesh.my_device.torch_device if multi else torch.device(kind)
        my_pp = mesh.my_mpmd_axis_index if multi else None
        tp_rank = mesh.axis_index("model") if multi and rc.tp > 1 else 0
        dp_rank = mesh.axis_index("data") if multi and rc.dp > 1 else 0
        sharded_opt = args.shard_optimizer and multi and rc.dp > 1
        from jaxpp_b200.utils import config as flags

        if rc.zb_defer_gb is not None and flags.zb_defer_bytes.value < 0:   # the configuration's own memory bound
            flags.zb_defer_bytes._override = int(rc.zb_defer_gb * 1e9)
        hyper = lt.Hyper(lr=args.lr, inplace_update=True, shard_optimizer=sharded_opt, clip_grad_norm=args.clip_grad_norm,
                         fp32_wgrad=rc.grad_bytes == 4)
        step_fn = lt.make_train_step(cfg, sched, hyper, dp_axis="data" if rc.dp > 1 else None, dp=rc.dp)
        state = lt.init_state(cfg, sched, device, my_rank=my_pp, tp_rank=tp_rank + 1000 * dp_rank * (rc.ep > 1), seed=args.seed)
        if sharded_opt:
            state = lt.shard_state_for_dp(cfg, state, rc.dp, dp_rank)
        specs = lt.state_specs(cfg, state, "data" if sharded_opt else None)
        jitted = jp.mpmd_jit_with_loop(step_fn, mesh, out_specs=(specs, jp.PartitionSpec()), name=rc.name)
        n_mb, mb_local = rc.n_microbatches, max(1, rc.microbatch // rc.dp)
        start, cursor = 0, 0
        compiled = None
        det = fault.FailureDetector(rank, world, interval_s=1.0, timeout_s=30.0).start() if multi else None
        if args.resume and args.ckpt_dir and ckpt.latest_step(args.ckpt_dir) is not None:
            tok = torch.zeros(n_mb, mb_local, cfg.seq, dtype=torch.int64, device=device)
            compiled = jitted.lower(state, tok, tok)
            target = compiled.out_shardings[0]
            state, extra = ckpt.load(args.ckpt_dir, None, target, mesh)
            start, cursor = int(extra["step"]), int(extra["cursor"])
            if rank == 0:
                print(f"resumed from step {start}", flush=True)
        metrics = StepMetrics(args.metrics, rc.global_batch * cfg.seq, rank=rank)
        for step in range(start, start + args.steps):
            gen = torch.Generator().manual_seed(args.seed * 1_000_003 + cursor * 131 + dp_rank)
            batch = torch.randint(0, cfg.vocab, (n_mb, mb_local, cfg.seq + 1), generator=gen).to(device)
            cursor += 1
            if det is not None:
                det.check()
            metrics.begin()
            scope = det.step_scope(step) if det is not None else _null()
            with scope:
                state, losses = jitted(state, batch[:, :, :-1].contiguous(), batch[:, :, 1:].contiguous())
                if device.type == "cuda":
                    # a fused kernel that ran out of its wait budget returned early and left outputs unwritten:
                    # raise inside the step scope, so that the failure record reaches the other ranks and nothing of
                    # this step is checkpointed
                    from jaxpp_b200.ops import native

                    native.raise_on_status(f"step {step}")
            lt_ = losses.local_tensor()
            rec = metrics.end(step, float(lt_.float().mean()) if lt_ is not None else None)
            if rank == 0:
                print(f"step {step}: {rec['step_ms']:.1f} ms, {rec['tokens_per_s']:.0f} tok/s", flush=True)
            if args.ckpt_dir and args.ckpt_every and (step + 1) % args.ckpt_every == 0:
                ckpt.save(args.ckpt_dir, step + 1, state, mesh, extra={"step": step + 1, "cursor": cursor, "config": rc.name})
        metrics.close()
        if det is not None:
            det.stop()

    distributed_main(run, backend=None if args.device is None else ("gloo" if args.device == "cpu" else "nccl"))


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


if __name__ == "__main__":
    main()
