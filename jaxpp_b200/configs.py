"""Named run configurations: model shape x mesh x schedule x batch, including the benchmark configurations.

Every configuration maps a GPU count to a mesh ``(mpmd, data, model)``, a schedule and a microbatching; the
batch sizes are *global* (sequences per step over all data-parallel replicas).
"""
from __future__ import annotations

import dataclasses
from typing import Callable


from . import api as jp
from .models import transformer as tf


@dataclasses.dataclass(frozen=True)
class RunConfig:
    name: str
    model: Callable[..., tf.ModelConfig]
    pp: int
    dp: int
    tp: int
    n_stages: int
    schedule: Callable[[int, int], jp.BaseSchedule]  # (n_stages, pp) -> schedule
    global_batch: int      # sequences per step
    microbatch: int        # sequences per microbatch (global, i.e. over all data-parallel ranks)
    ep: int = 1            # expert parallel size (uses the data axis)
    recompute: bool = False
    description: str = ""
    # what the configuration needs to fit 180 GB (see memory_plan): bytes per parameter of the gradient accumulators
    # (4 = fp32, 2 = bf16) and, for schedules that split the backward, the bound on the operands that deferred
    # weight-gradient GEMMs keep alive per (stage, microbatch), in GB (None = no bound)
    grad_bytes: int = 4
    zb_defer_gb: float | None = None

    @property
    def n_gpus(self) -> int:
        return self.pp * self.dp * self.tp

    @property
    def n_microbatches(self) -> int:
        return self.global_batch // self.microbatch

    def model_config(self, **over) -> tf.ModelConfig:
        kw = dict(n_stages=self.n_stages, tp=self.tp, recompute=self.recompute)
        if self.ep > 1:
            kw["ep"] = self.ep
        kw.update(over)
        return self.model(**kw)

    def make_schedule(self) -> jp.BaseSchedule:
        return self.schedule(self.n_stages, self.pp)

    def mesh_shape(self) -> dict:
        return {"mpmd": self.pp, "data": self.dp, "model": self.tp}


_std = lambda s, p: jp.Std1F1B(p)
_inter = lambda s, p: jp.Interleaved1F1B(s, p)
_zb = lambda s, p: jp.ZeroBubble(p)
_dpv = lambda s, p: jp.DualPipeV(s, p)

CONFIGS: dict[str, RunConfig] = {c.name: c for c in [
    RunConfig("encoder_cpu_pp2", tf.bert_example, 2, 1, 1, 2, _std, 32, 8,
              description="4-layer BERT-style encoder, fp32, 2 stages on 2 CPU ranks, Std1F1B, 4 microbatches of 8x128"),
    RunConfig("gpt2xl_pp2dp4", tf.gpt2_xl, 2, 4, 1, 2, _std, 64, 4,
              description="GPT-2-XL shape, PP2 x DP4, Std1F1B, 16 microbatches of 4 (1 sequence per replica)"),
    RunConfig("llama7b_pp4tp2", tf.llama2_7b, 4, 1, 2, 8, _inter, 128, 4,
              description="Llama-2-7B shape, PP4 x TP2, Interleaved1F1B with 2 virtual stages, 32 microbatches of 4 (headline)"),
    RunConfig("llama7b_pp2tp2", tf.llama2_7b, 2, 1, 2, 4, _inter, 64, 4, description="4-GPU slice of the headline layout"),
    RunConfig("llama7b_tp2", tf.llama2_7b, 1, 1, 2, 1, _std, 32, 4, description="2-GPU slice of the headline layout"),
    RunConfig("llama7b_single", tf.llama2_7b, 1, 1, 1, 1, _std, 16, 1, description="one GPU, 16 microbatches of 1"),
    RunConfig("mixtral8x7b_pp2ep4", tf.mixtral_8x7b, 2, 4, 1, 4, _dpv, 64, 8, ep=4, recompute=True, zb_defer_gb=8.0,
              description="Mixtral-8x7B shape, PP2 x EP4 (experts over the data axis), DualPipeV, microbatches of 2 per replica; "
                          "blocks recomputed in backward: without it the memory plan exceeds 180 GB per GPU"),
    RunConfig("llama70b_pp4tp2", tf.llama2_70b, 4, 1, 2, 4, _zb, 64, 1, recompute=True, grad_bytes=2, zb_defer_gb=2.0,
              description="Llama-2-70B shape, PP4 x TP2, ZeroBubble, 64 microbatches of 1, full activation recompute; 8.8 B "
                          "parameters per GPU leave no room for fp32 gradient accumulators (bf16 ones) nor for the operands of "
                          "every deferred weight gradient (at most 2 GB per task stay alive, the rest run with the activation "
                          "gradients)"),
]}


def choose_stage_layers(cfg: tf.ModelConfig, schedule, pp: int, tokens_per_microbatch: int, mode: str = "auto"):
    """Stage sizes for ``cfg`` under ``schedule``: ``"equal"`` (None: the model's default), a comma-separated list of
    sizes in blocks (multiples of 0.5), or ``"auto"``: the split that evens out the pipeline ranks' work, counted in
    FLOPs -- or in kernels when the configuration is bound by launches (:func:`transformer.launch_bound`)."""
    n_stages = cfg.n_stages
    if mode == "equal" or n_stages <= 1:
        return None
    if mode != "auto":
        return tuple(float(x) for x in mode.split(","))
    attn_share, head_extra, first_extra = tf.stage_cost_model(cfg)
    if tf.launch_bound(cfg, tokens_per_microbatch):
        attn_share, head_extra = 0.5, 0.1   # stages cost their number of kernels: the head is a dozen launches
    return tf.balanced_stage_layers(cfg.n_layers, n_stages, schedule.get_mpmd_idx, pp, first_extra=first_extra,
                                    last_extra=head_extra, attn_share=attn_share, max_shift=max(1.0, min(3.0, head_extra)))


def get(name: str) -> RunConfig:
    if name not in CONFIGS:
        raise KeyError(f"unknown configuration {name!r}; available: {sorted(CONFIGS)}")
    return CONFIGS[name]


# =============================================================================================
# memory plan: does a configuration fit the 180 GB of a B200?
# =============================================================================================
HBM_BYTES = 180e9


def peak_live_microbatches(schedule: jp.BaseSchedule, n_microbatches: int) -> list[int]:
    """Per pipeline rank: the largest number of (stage, microbatch) forward activations alive at once, i.e. forwards
    run whose backward (the weight-gradient half, when the backward is split) has not run yet, in the rank's task
    order."""
    from .schedules import FusedTask
    from .types import TaskType

    releases = TaskType.BWD_W if schedule.is_partial_bwd else TaskType.BWD
    peaks = []
    for row in schedule.tasks(n_microbatches):
        live = peak = 0
        for unit in row:
            if unit is None:
                continue
            for t in (unit if isinstance(unit, FusedTask) else (unit,)):
                if t.fwd_or_bwd is TaskType.FWD:
                    live += 1
                    peak = max(peak, live)
                elif t.fwd_or_bwd is releases:
                    live -= 1
        peaks.append(peak)
    return peaks


def peak_deferred_weight_gradients(schedule: jp.BaseSchedule, n_microbatches: int) -> list[int]:
    """Per pipeline rank of a split-backward schedule: the largest number of (stage, microbatch) activation-gradient
    tasks whose weight-gradient task has not run yet, in the rank's task order.  The operands of the deferred
    weight-gradient GEMMs (activation gradients and, with recompute, the recomputed inputs of every linear) stay alive
    for each of them.  The first stage's backward is never split and does not count."""
    from .schedules import FusedTask
    from .types import TaskType

    out = []
    for row in schedule.tasks(n_microbatches):
        pending: set = set()
        peak = 0
        for unit in row:
            if unit is None:
                continue
            for t in (unit if isinstance(unit, FusedTask) else (unit,)):
                if t.fwd_or_bwd is TaskType.BWD_I and t.stage_id != 0:
                    pending.add((t.stage_id, t.mubatch_idx))
                    peak = max(peak, len(pending))
                elif t.fwd_or_bwd is TaskType.BWD_W:
                    pending.discard((t.stage_id, t.mubatch_idx))
        out.append(peak)
    return out


def memory_plan(rc: RunConfig, shard_optimizer: bool = False, grad_bytes: int | None = None,
                zb_defer_bytes: float | None = -1.0) -> dict:
    """Estimated bytes per GPU of the busiest pipeline rank: bf16 parameters, fp32 master weights and Adam moments
    (1/dp of them with ``shard_optimizer``), gradient accumulators (``grad_bytes`` per parameter: 4, or 2 with bf16
    accumulation), the activations that the schedule keeps alive (per block: what the backward of the fused kernels
    needs; with recompute only the block inputs plus one block's working set) and, for schedules that split the
    backward, the operands that deferred weight-gradient GEMMs hold between the two halves (bounded per (stage,
    microbatch) by ``zb_defer_bytes`` when given, see ``JAXPP_B200_ZB_DEFER_BYTES``).  An estimate for sizing, not an
    allocator trace."""
    grad_bytes = rc.grad_bytes if grad_bytes is None else grad_bytes
    if zb_defer_bytes is not None and zb_defer_bytes < 0:      # default: the configuration's own bound
        zb_defer_bytes = None if rc.zb_defer_gb is None else rc.zb_defer_gb * 1e9
    cfg = rc.model_config()
    d, f, hd = cfg.d_model, cfg.ffn, cfg.head_dim
    tp, ep = rc.tp, max(1, rc.ep)
    attn_w = d * (cfg.n_heads + 2 * cfg.n_kv_heads) * hd + cfg.n_heads * hd * d
    if cfg.n_experts:
        mlp_w = 3 * d * f * cfg.n_experts / ep + d * cfg.n_experts          # experts over the expert axis + router
    else:
        mlp_w = (3 if cfg.family in ("llama", "mixtral") else 2) * d * f
    per_layer = (attn_w + (mlp_w if cfg.n_experts else mlp_w)) / tp if not cfg.n_experts else attn_w / tp + mlp_w
    layers_per_rank = cfg.n_layers / rc.pp
    embed = cfg.padded_vocab * d                                           # embedding on the first rank, head on the last
    params = layers_per_rank * per_layer + embed
    weights = 2 * params
    optimizer = 12 * params
    if shard_optimizer and rc.dp > 1:
        # only replicas over the data axis are sliced; experts sharded over that axis stay whole on their owner
        experts = layers_per_rank * 3 * d * f * cfg.n_experts / ep if cfg.n_experts else 0.0
        optimizer = 12 * (experts + (params - experts) / rc.dp)
    grads = grad_bytes * params
    # activations of one block for one microbatch, bytes per local token (bf16 unless noted)
    tokens = (rc.microbatch // rc.dp) * cfg.seq
    heads_local = (cfg.n_heads + 2 * cfg.n_kv_heads) * hd / tp
    ffn_local = (f / tp) * (cfg.top_k if cfg.n_experts else 1)
    block = 2 * (d / tp            # block input, sequence-sharded under tensor parallelism
                 + d / tp          # normalised input (sharded, re-gathered by the fused kernel)
                 + heads_local     # q, k, v after the split
                 + cfg.n_heads * hd / tp   # attention output
                 + d / tp          # residual / second norm input
                 + d / tp          # second normalised input
                 + (2 if cfg.family in ("llama", "mixtral") else 1) * ffn_local   # gate | up (or the GELU input)
                 + ffn_local)      # activation output
    block += 4 * cfg.n_heads / tp  # log-sum-exp, fp32
    live = max(peak_live_microbatches(rc.make_schedule(), rc.n_microbatches))
    layers_per_stage = cfg.n_layers / rc.n_stages
    if rc.recompute:
        acts = tokens * (live * layers_per_stage * 2 * d / tp + block)
    else:
        acts = tokens * live * layers_per_stage * block
    logits = tokens / tp * cfg.padded_vocab * (2 + 4)                       # bf16 logits + fp32 gradient of one microbatch
    # operands of the weight-gradient GEMMs of one block for one microbatch (bf16): (dy, x) of the four linears, in
    # the forms the tensor-parallel ops keep them (sequence-sharded inputs of the column-parallel ones)
    sched = rc.make_schedule()
    deferred = 0.0
    if sched.is_partial_bwd:
        wgrad_block = 2 * tokens * (heads_local + d / tp            # qkv: dy [T, heads_local], x shard
                                    + d + cfg.n_heads * hd / tp     # wo: gathered dy [T, d], x [T, heads/tp]
                                    + (2 if cfg.family in ("llama", "mixtral") else 1) * ffn_local + d / tp   # up
                                    + d + ffn_local)                # down
        per_task = wgrad_block * layers_per_stage
        if zb_defer_bytes is not None and zb_defer_bytes >= 0:
            per_task = min(per_task, zb_defer_bytes)
        deferred = per_task * max(peak_deferred_weight_gradients(sched, rc.n_microbatches))
    total = weights + optimizer + grads + acts + logits + deferred
    return {"config": rc.name, "params_per_gpu": params, "weights": weights, "optimizer": optimizer, "grads": grads,
            "activations": acts, "logits": logits, "deferred_wgrad_operands": deferred, "live_stage_microbatches": live,
            "total": total, "fits": total < 0.92 * HBM_BYTES}


def _main():
    import argparse

    ap = argparse.ArgumentParser(description="per-GPU memory estimate of every named configuration")
    ap.add_argument("--shard-optimizer", action="store_true")
    ap.add_argument("--bf16-grads", action="store_true", help="2-byte gradient accumulators")
    ap.add_argument("--zb-defer-gb", type=float, default=None, help="bound on deferred weight-gradient operands per task")
    args = ap.parse_args()
    gb = lambda x: f"{x / 1e9:7.1f}"
    print(f"{'configuration':<22}{'params/GPU':>11}{'weights':>9}{'optim':>8}{'grads':>8}{'acts':>8}{'logits':>8}{'deferred':>9}{'total GB':>10}  fits 180 GB")
    for rc in CONFIGS.values():
        if rc.name.startswith("encoder"):
            continue
        m = memory_plan(rc, args.shard_optimizer, 2 if args.bf16_grads else None,
                        -1.0 if args.zb_defer_gb is None else args.zb_defer_gb * 1e9)
        print(f"{rc.name:<22}{m['params_per_gpu'] / 1e9:>10.2f}B{gb(m['weights']):>9}{gb(m['optimizer']):>8}{gb(m['grads']):>8}"
              f"{gb(m['activations']):>8}{gb(m['logits']):>8}{gb(m['deferred_wgrad_operands']):>9}{gb(m['total']):>10}  {'yes' if m['fits'] else 'NO'}")


if __name__ == "__main__":
    _main()
