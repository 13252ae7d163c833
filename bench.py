#!/usr/bin/env python
"""Headline benchmark: training tokens/s of a Llama-2-7B-shape decoder, bf16, AdamW, synthetic data.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Weak scaling: every GPU contributes 16 sequences of 4096 tokens per step.  N=8 is the headline layout
(PP=4 x TP=2, Interleaved1F1B with 2 virtual stages per rank, 32 microbatches of 4 sequences); smaller N
keep the model and the per-GPU batch and shrink the mesh: N=4 PP2xTP2, N=2 TP2, N=1 a single device
(16 microbatches of 1 sequence so that activations fit beside 7B of optimizer state).  ``--config NAME`` runs
any other named configuration (GPT-2-XL PP2xDP4, Mixtral-8x7B PP2xEP4, Llama-2-70B PP4xTP2) the same way.

Prints ONE JSON line from rank 0.  ``value`` is device-timed (CUDA events around K steps, max over ranks);
``e2e`` repeats the measurement through the public API with a host->device copy of the step's token ids
from pinned memory and a device->host read of the loss in every step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None,
                    help="a named run configuration of jaxpp_b200.configs (gpt2xl_pp2dp4, mixtral8x7b_pp2ep4, llama70b_pp4tp2, "
                         "...) instead of the headline layout for --gpus; its GPU count must equal --gpus")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; invalid as a result)")
    ap.add_argument("--seqs-per-gpu", type=int, default=16, help="headline layouts: sequences per GPU and step (weak scaling)")
    ap.add_argument("--nccl-only", action="store_true", help="baseline: NCCL collectives instead of fused kernels")
    ap.add_argument("--stage-layers", default="auto",
                    help="blocks per pipeline stage: 'equal', 'auto' (balance the pipeline ranks, counting the output "
                         "projection and loss of the last stage) or a comma-separated list (entries may end in .5)")
    ap.add_argument("--shard-optimizer", action="store_true", help="optimizer state as 1/dp slices (data-parallel configs)")
    ap.add_argument("--timeline", default=None, help="write a per-rank, per-task-kind timeline of one step to this file")
    ap.add_argument("--op-times", default=None,
                    help="write per-op device times of one extra step (CUDA events around every op call) to this file")
    ap.add_argument("--bf16-grads", action="store_true",
                    help="accumulate weight gradients in bf16 instead of fp32 (2 bytes per parameter less; for models whose "
                         "fp32 optimizer state leaves no room)")
    ap.add_argument("--zb-defer-gb", type=float, default=None,
                    help="zero-bubble schedules: bytes (GB) of operands that deferred weight-gradient GEMMs may keep alive per "
                         "(stage, microbatch); the rest of the weight gradients run with the activation gradients")
    ap.add_argument("--no-grad-overlap", action="store_true",
                    help="run the data-parallel gradient collectives after the loop instead of from the last backward tasks")
    ap.add_argument("--smoke-cpu", action="store_true",
                    help="harness check only: the same script on CPU ranks over gloo with a shrunken model (not a result)")
    ap.add_argument("--p2p", default=None, choices=[None, "torch", "native"], help="point-to-point backend between stages")
    return ap.parse_args()


# headline layouts: n_gpus -> named configuration (all the Llama-2-7B shape; 16 sequences of 4096 per GPU)
HEADLINE = {1: "llama7b_single", 2: "llama7b_tp2", 4: "llama7b_pp2tp2", 8: "llama7b_pp4tp2"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm():
    # The reference is JAX-based: its package installs from the offline wheelhouse only with --no-deps and
    # cannot be imported because jax / jaxlib / cupy are neither installed nor in the wheelhouse.
    print(json.dumps({"impl": "reference", "unavailable": "reference needs jax[cuda12]+cupy, absent from image and wheelhouse "
                      "(pip --no-index: no matching distribution for jax); `import jaxpp` fails with ModuleNotFoundError: jax"}))


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm()

    import dataclasses

    import torch
    import torch.distributed as dist

    import jaxpp_b200 as jp
    from jaxpp_b200 import configs
    from jaxpp_b200.models import lm_trainer as lt
    from jaxpp_b200.models import transformer as tf
    from jaxpp_b200.ops import native
    from jaxpp_b200.parallel import fused, symm
    from jaxpp_b200.utils import config, timeline

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n = args.gpus
    if world != n:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n}")
    headline = args.config is None
    if headline and n not in HEADLINE:
        raise SystemExit(f"supported GPU counts: {sorted(HEADLINE)}")
    rc = configs.get(HEADLINE[n] if headline else args.config)
    if rc.n_gpus != n:
        raise SystemExit(f"{rc.name} runs on {rc.n_gpus} GPUs, not {n}")
    cuda = not args.smoke_cpu
    if cuda:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=device)
        native.load()
    else:
        device = torch.device("cpu")
        if world > 1:
            dist.init_process_group("gloo")

    class Ev:   # a CUDA event on the current stream, or a wall-clock stamp on CPU ranks
        def __init__(self):
            self.e = torch.cuda.Event(enable_timing=True) if cuda else None
            self.t = 0.0

        def record(self):
            if cuda:
                self.e.record()
            else:
                self.t = time.perf_counter()

        def elapsed_time(self, other):
            return self.e.elapsed_time(other.e) if cuda else (other.t - self.t) * 1e3

    def dev_sync():
        if cuda:
            torch.cuda.synchronize()
    if args.nccl_only:
        config.use_fused_collectives._override = False
    if args.p2p:
        config.p2p_backend._override = args.p2p
    config.transfer_done_delay._override = 2  # release sent activations two sends later instead of at step end
    zb_defer_gb = args.zb_defer_gb if args.zb_defer_gb is not None else rc.zb_defer_gb   # the configuration's own bound
    if zb_defer_gb is not None:
        config.zb_defer_bytes._override = int(zb_defer_gb * 1e9)
    bf16_grads = args.bf16_grads or rc.grad_bytes == 2
    if args.no_grad_overlap:
        config.overlap_grad_reduce._override = False

    pp, tp, dp = rc.pp, rc.tp, rc.dp
    n_stages = rc.n_stages
    seqs = args.seqs_per_gpu * n if headline else rc.global_batch
    mb = rc.microbatch
    n_mb = seqs // mb
    mb_local = max(1, mb // dp)
    schedule = rc.make_schedule()
    cfg = rc.model_config()
    if args.layers:
        cfg = dataclasses.replace(cfg, n_layers=args.layers)
    if args.smoke_cpu:
        over = dict(vocab=256, d_model=64, n_layers=2 * n_stages, n_heads=4, n_kv_heads=2 if cfg.n_kv_heads != cfg.n_heads else 4,
                    ffn=128, seq=32, dtype=torch.float32)
        if rc.ep > 1:
            over.update(n_experts=2 * rc.ep, capacity_factor=4.0)
        cfg = dataclasses.replace(cfg, **over)
    sizes = configs.choose_stage_layers(cfg, schedule, pp, mb_local * cfg.seq, args.stage_layers)
    if sizes is not None:
        cfg = dataclasses.replace(cfg, stage_layers=sizes)
    mesh = jp.MpmdMesh.create({"mpmd": pp, "data": dp, "model": tp}, kind="cuda" if cuda else "cpu", multi_process=world > 1)
    if world > 1:
        for axis, size in (("model", tp), ("data", dp)):
            if size > 1:
                mesh.axis_group(axis)  # created collectively, up front
    my_pp = mesh.my_mpmd_axis_index if world > 1 else None
    tp_rank = mesh.axis_index("model") if world > 1 and tp > 1 else 0
    dp_rank = mesh.axis_index("data") if world > 1 and dp > 1 else 0

    sharded_opt = args.shard_optimizer and dp > 1
    hyper = lt.Hyper(shard_optimizer=sharded_opt, fp32_wgrad=not bf16_grads)
    step_fn = lt.make_train_step(cfg, schedule, hyper, dp_axis="data" if dp > 1 else None, dp=dp)
    jitted = jp.mpmd_jit_with_loop(step_fn, mesh, name=f"{rc.name}_train_step")
    # expert weights differ between the ranks of the expert axis; everything else is replicated over the data axis
    state = lt.init_state(cfg, schedule, device, my_rank=my_pp, tp_rank=tp_rank + 1000 * dp_rank * (rc.ep > 1), seed=0)
    if sharded_opt:
        state = lt.shard_state_for_dp(cfg, state, dp, dp_rank)

    g = torch.Generator().manual_seed(1234 + dp_rank)
    host_tokens = [torch.randint(0, cfg.vocab, (n_mb, mb_local, cfg.seq + 1), generator=g) for _ in range(2)]
    if cuda:
        host_tokens = [t.pin_memory() for t in host_tokens]
    tokens_per_step = seqs * cfg.seq
    h2d_bytes = n_mb * mb_local * (cfg.seq + 1) * 8

    def load_batch(i):
        t = host_tokens[i % 2].to(device, non_blocking=True)
        return t[:, :, :-1].contiguous(), t[:, :, 1:].contiguous()

    def sync_all():
        dev_sync()
        if world > 1:
            dist.barrier()
            dev_sync()

    def read_loss(losses):
        t = losses.local_tensor()
        return float(t.mean().item()) if t is not None else None

    def mean_over_ranks(v):
        """Mean of a per-rank value over the ranks that have one (the ranks of the last pipeline stage)."""
        if world == 1:
            return v
        t = torch.tensor([v if v is not None else 0.0, 0.0 if v is None else 1.0], device=device, dtype=torch.float64)
        dist.all_reduce(t)
        return float(t[0] / t[1]) if float(t[1]) > 0 else None

    tok, lab = load_batch(0)
    loss_val = first_loss = None
    for i in range(args.warmup):
        state, losses = jitted(state, tok, lab)
        loss_val = read_loss(losses)
        if i == 0:
            first_loss = loss_val
    sync_all()
    if cuda:
        torch.cuda.reset_peak_memory_stats()

    # ---- device-timed region: K steps, inputs resident -------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0 and cuda:
        sampler.start()
    native.LAUNCHES[0] = 0
    e0, e1 = Ev(), Ev()
    sync_all()
    e0.record()
    for i in range(args.steps):
        state, losses = jitted(state, tok, lab)
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1) / args.steps
    launches = native.LAUNCHES[0]
    clocks = sampler.stop() if rank == 0 else None
    status = native.read_status() if cuda else 0

    # ---- end-to-end region: H2D of the step's tokens + D2H of its loss, every step ----------------------------------
    sync_all()
    t0 = time.perf_counter()
    for i in range(args.steps):
        tok, lab = load_batch(i)
        state, losses = jitted(state, tok, lab)
        lv = read_loss(losses)
        loss_val = lv if lv is not None else loss_val
    sync_all()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    peak_mem = torch.cuda.max_memory_allocated() / 1e9 if cuda else 0.0
    from jaxpp_b200.runtime import executor as _ex
    if _ex.LIVE_REPORT:   # JAXPP_B200_TRACK_LIVE_BYTES=1: what the step's environment held at its fullest
        rep = _ex.LIVE_REPORT[-1]
        state_bytes = sum(t.untyped_storage().nbytes() for t in torch.utils._pytree.tree_leaves(state) if isinstance(t, torch.Tensor))
        print(f"[live rank {rank}] peak {rep['bytes'] / 1e6:.1f} MB in {rep['n_values']} values before {rep['before']}; "
              f"state {state_bytes / 1e6:.1f} MB; largest: "
              + "; ".join(f"%{v} {sh} {dt} {b / 1e6:.2f}MB" for b, v, sh, dt in rep["largest"]), file=sys.stderr, flush=True)
        if os.environ.get("JAXPP_B200_TRACK_LIVE_BYTES_SHAPES") == "1" and rank == 0:
            import collections
            cnt = collections.Counter((sh, dt) for b, v, sh, dt in rep["all"])
            print("[live shapes] " + "; ".join(f"{sh} {dt} x{c}" for (sh, dt), c in cnt.most_common(30)), file=sys.stderr, flush=True)

    # ---- bubble and timeline: one extra step with per-task CUDA events ---------------------------------------------------
    compiled = jitted.lower(state, tok, lab)
    leaves, *_ = jitted._prepare((state, tok, lab), {})
    sync_all()
    b0, b1 = Ev(), Ev()
    b0.record()
    out = compiled(leaves, record_events=True)
    b1.record()
    dev_sync()
    step_ms_b = b0.elapsed_time(b1)
    busy = compiled.last_states[0].busy_ms() if world > 1 else sum(s.busy_ms() for s in compiled.last_states)
    bubble = max(0.0, 1.0 - busy / step_ms_b) if cuda else 0.0
    if args.timeline and cuda:
        text = "\n".join(timeline.format_summary(
            f"process {rank} (pipeline rank {st.rank}, tp {tp_rank}, dp {dp_rank})", timeline.summarise_events(st.events, b0.e, b1.e))
            for st in compiled.last_states)
        texts = [text]
        if world > 1:
            texts = [None] * world
            dist.all_gather_object(texts, text)
        if rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(args.timeline)), exist_ok=True)
            with open(args.timeline, "w") as f:
                f.write(f"# one step of {rc.name} on {n} GPUs with per-task CUDA events (stage sizes {cfg.stage_sizes}); "
                        "'idle before' = compute stream idle in front of a task (waiting for another rank)\n")
                f.write("\n\n".join(texts) + "\n")

    if args.op_times and cuda:
        from jaxpp_b200.utils import optimes

        sync_all()
        with optimes.collecting():
            o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            o0.record()
            compiled(leaves)
            o1.record()
            torch.cuda.synchronize()
            rows = optimes.table()
        text = optimes.format_table(rows, o0.elapsed_time(o1),
                                    f"process {rank} (pipeline rank {my_pp if my_pp is not None else 0}, tp {tp_rank}, dp {dp_rank})")
        texts = [text]
        if world > 1:
            texts = [None] * world
            dist.all_gather_object(texts, text)
        if rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(args.op_times)), exist_ok=True)
            with open(args.op_times, "w") as f:
                f.write(f"# per-op device time of one step of {rc.name} on {n} GPUs: CUDA events around every op call of every "
                        f"task, under the conditions of the timed run (uninstrumented step: {ms:.1f} ms)\n")
                f.write("\n\n".join(texts) + "\n")

    canary_lines = symm.canary_reports() if cuda else []
    canaries_ok = not canary_lines
    if canary_lines:
        print(f"[rank {rank}] " + " | ".join(canary_lines), file=sys.stderr, flush=True)
    fallbacks = fused.FALLBACKS[0]
    loss_val, first_loss = mean_over_ranks(loss_val), mean_over_ranks(first_loss)
    bubbles, peaks = [bubble], [peak_mem]
    if world > 1:
        allb = [torch.zeros(2, device=device, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(allb, torch.tensor([bubble, peak_mem], device=device, dtype=torch.float64))
        bubbles, peaks = [float(x[0]) for x in allb], [float(x[1]) for x in allb]
        t = torch.tensor([ms, e2e_ms, bubble, float(launches), float(status), float(fallbacks), float(not canaries_ok)],
                         device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, bubble, launches, status, fallbacks, bad_canary = (float(x) for x in t.tolist())
        canaries_ok = not bad_canary

    if rank == 0:
        value = tokens_per_step / (ms / 1e3)
        flops = cfg.flops_per_token() * tokens_per_step   # model FLOPs: recomputed forwards are not counted
        peak = 1412.0e12
        try:
            peaks_json = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
            peak = float(peaks_json.get("bf16_tflops_sustained", 1412.0)) * 1e12
        except Exception:
            pass
        par = "".join(f"{k}{v}" for k, v in (("pp", pp), ("dp", dp), ("tp", tp)) if v > 1 or k == "pp")
        if rc.ep > 1:
            par = par.replace(f"dp{dp}", f"ep{rc.ep}")
        vstages = n_stages // pp
        metric = ("train tokens/s, Llama-7B-shape PP4xTP2 on 8xB200 (max over ranks); bubble %" if headline
                  else f"train tokens/s, {rc.name} on {n}xB200 (max over ranks); bubble %")
        out = {
            "metric": metric,
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"name": rc.name,
                       "model": f"{rc.model.__name__} ({cfg.n_layers} layers, d_model {cfg.d_model}, seq {cfg.seq})",
                       "global_batch": seqs, "seq_len": cfg.seq, "microbatches": n_mb, "microbatch_size": mb,
                       "parallelism": par + (f" v={vstages}" if vstages > 1 else ""),
                       "schedule": type(schedule).__name__, "stage_layers": list(cfg.stage_sizes),
                       "recompute": bool(cfg.recompute),
                       "optimizer": "AdamW fp32 master, fused kernel" + (", state sharded over dp" if sharded_opt else "")
                                    + (", bf16 gradient accumulators" if bf16_grads else ", fp32 gradient accumulators"),
                       "grad_reduce_overlap": bool(config.overlap_grad_reduce.value) and dp > 1,
                       "zb_defer_bytes": int(config.zb_defer_bytes.value),
                       "l2": "inputs exceed L2 (weights and activations are GBs per step)",
                       "fused_collectives": bool(config.use_fused_collectives.value) and (tp > 1 or dp > 1),
                       "p2p": config.p2p_backend.value},
            "clocks": clocks,
            "e2e": {"value": round(tokens_per_step / (e2e_ms / 1e3), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_ms, 3)},
            "gpu_launches": int(launches),
            "bubble_pct": round(100 * bubble, 2),
            "ideal_bubble_pct": round(100 * schedule.ideal_bubble_fraction(n_mb), 2),
            "mfu_of_measured_sustained_peak": round(flops / (ms / 1e3) / (peak * n), 4),
            "bubble_pct_per_rank": [round(100 * b, 2) for b in bubbles],
            "peak_mem_gb_per_rank": [round(x, 1) for x in peaks],
            "first_step_loss": first_loss, "ln_vocab": round(math.log(cfg.vocab), 3),
            "final_loss": loss_val, "kernel_status": int(status),
            "fused_fallbacks": int(fallbacks), "canaries_ok": bool(canaries_ok),
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
