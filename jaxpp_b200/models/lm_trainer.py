"""Language-model train step (mixed precision, AdamW) on top of the pipelining API, plus state set-up.

State layout (a pytree that the step maps to a new pytree of the same structure, as the reference's
steps do with their Flax ``TrainState``):

    {"params": bf16 compute copy, "master": fp32 weights, "m": Adam first moment, "v": second moment,
     "step": int64 scalar}

The step casts nothing inside the microbatch loop: the compute copy is kept up to date by the fused
AdamW kernel, weight gradients leave the GEMM epilogue in fp32, are summed over microbatches by
``treduce`` and reach AdamW with the 1/tokens normalisation folded into its ``grad_scale``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable

import torch
from torch.utils import _pytree as pytree

from .. import api as jp
from ..core import ShapeDtypeStruct
from ..ops import core as ops
from ..parallel import tp as tpops
from . import transformer as tf


@dataclasses.dataclass(frozen=True)
class Hyper:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    fp32_wgrad: bool = True
    inplace_update: bool = True  # the step consumes the state it is given (donation)


def stage_of_layer(cfg: tf.ModelConfig, layer: int) -> int:
    return layer // cfg.layers_per_stage


def owner_ranks(cfg: tf.ModelConfig, schedule) -> dict:
    """Pipeline rank of every parameter group: ``{"embed": r, "head": r, layer index: r}``."""
    out: dict[Any, int] = {i: int(schedule.get_mpmd_idx(stage_of_layer(cfg, i))) for i in range(cfg.n_layers)}
    out["embed"] = int(schedule.get_mpmd_idx(0))
    out["head"] = int(schedule.get_mpmd_idx(cfg.n_stages - 1))
    return out


def init_state(cfg: tf.ModelConfig, schedule, device, my_rank: int | None = None, tp_rank: int = 0, seed: int = 0) -> dict:
    """Training state for pipeline rank ``my_rank`` (``None`` = everything, for single-process runs).

    Parameter groups owned by other ranks are present as :class:`ShapeDtypeStruct` leaves so that the
    pytree has the same structure on every process.
    """
    owners = owner_ranks(cfg, schedule)
    mine = lambda key: my_rank is None or owners[key] == my_rank
    tied_extra = cfg.tie_embeddings and my_rank is not None and owners["head"] == my_rank
    full = tf.init_params(cfg, "meta", seed, tp_rank)  # structure and shapes only
    local_layers = [i for i in range(cfg.n_layers) if mine(i)]
    real = tf.init_params(cfg, device, seed, tp_rank, layers=local_layers, with_embed=mine("embed") or tied_extra,
                          with_head=mine("head"))

    def pick(path_keys, meta_leaf):
        node = real
        for k in path_keys:
            if not isinstance(node, dict) or k not in node:
                return None
            node = node[k]
        return node

    def build(tree, path=()):
        if isinstance(tree, dict):
            return {k: build(v, path + (k,)) for k, v in tree.items()}
        got = pick(path, tree)
        return got if got is not None else ShapeDtypeStruct(tuple(tree.shape), tree.dtype)

    params = build(full)

    def like(p, dtype, fill=None):
        if isinstance(p, ShapeDtypeStruct):
            return ShapeDtypeStruct(p.shape, dtype)
        if fill is None:
            return p.detach().to(dtype).clone()
        return torch.zeros_like(p, dtype=dtype)

    is_leaf = lambda x: isinstance(x, ShapeDtypeStruct)
    master = pytree.tree_map(lambda p: like(p, torch.float32), params, is_leaf=is_leaf)
    m = pytree.tree_map(lambda p: like(p, torch.float32, 0), params, is_leaf=is_leaf)
    v = pytree.tree_map(lambda p: like(p, torch.float32, 0), params, is_leaf=is_leaf)
    return {"params": params, "master": master, "m": m, "v": v, "step": torch.zeros((), dtype=torch.int64, device=device)}


def make_train_step(cfg: tf.ModelConfig, schedule, hyper: Hyper = Hyper(), dp_axis: str | None = None,
                    dp: int = 1) -> Callable:
    """``step(state, tokens, labels) -> (state, losses)`` with ``tokens``/``labels`` of shape
    [n_microbatches, microbatch, seq]; ``losses[i]`` is the mean token loss of microbatch ``i`` over this
    device's tokens."""

    def step(state, tokens, labels):
        params = state["params"]
        n_mb, mb, seq = tokens.shape
        tokens_per_mb_local = mb * seq // cfg.tp
        total_tokens = n_mb * mb * seq * dp
        rope = tf.rope_tables(cfg, tokens.device) if cfg.family in ("llama", "mixtral") else None

        def body(batch):
            tok, lab = batch

            def loss_fn(p):
                return tf.lm_loss(cfg, p, tok, lab, rope)

            prev = ops.WGRAD_DTYPE[0]
            ops.WGRAD_DTYPE[0] = torch.float32 if hyper.fp32_wgrad else None
            try:
                loss, grads = jp.value_and_grad(loss_fn, grad_dtype=torch.float32 if hyper.fp32_wgrad else None)(params)
            finally:
                ops.WGRAD_DTYPE[0] = prev
            return loss / tokens_per_mb_local, grads

        losses, grads = jp.treduce(body, (tokens, labels), schedule=schedule)
        grads = tf.sync_replicated_grads(cfg, grads)
        if dp_axis is not None and dp > 1:
            grads = tf.sync_data_parallel_grads(cfg, grads, dp_axis)
        new_step = state["step"] + 1

        def update(p, master, g, m, v):
            pm, mm, vm, lp = ops.adamw(master, g, m, v, new_step, hyper.lr, hyper.beta1, hyper.beta2, hyper.eps,
                                       hyper.weight_decay if p.dim() > 1 else 0.0, 1.0 / total_tokens, p.dtype,
                                       p if hyper.inplace_update else None, hyper.inplace_update)
            return lp, pm, mm, vm

        flat_p, spec = pytree.tree_flatten(params)
        flat = [update(p, ma, g, m, v) for p, ma, g, m, v in zip(
            flat_p, pytree.tree_leaves(state["master"]), pytree.tree_leaves(grads), pytree.tree_leaves(state["m"]),
            pytree.tree_leaves(state["v"]))]
        unf = lambda k: pytree.tree_unflatten([f[k] for f in flat], spec)
        new_state = {"params": unf(0), "master": unf(1), "m": unf(2), "v": unf(3), "step": new_step}
        return new_state, losses

    return step


def param_specs(cfg: tf.ModelConfig, params_like: dict) -> dict:
    """PartitionSpec of every parameter (global view = concatenation of the shards along the sharded dim).

    Note that the global row order of ``wqkv`` / ``w_up`` is shard-major ([q_r | k_r | v_r] per rank): restoring a
    checkpoint with a different tensor-parallel size needs the rows regrouped (``transformer.shard_layer_for_tp``
    defines the canonical-to-shard mapping)."""
    P = jp.PartitionSpec
    tp, ep = cfg.tp_axis if cfg.tp > 1 else None, cfg.ep_axis if cfg.ep > 1 else None
    col = {"wqkv": P(tp, None), "w_up": P(tp, None), "b_qkv": P(tp), "b_up": P(tp)}
    row = {"wo": P(None, tp), "w_down": P(None, tp)}
    exp = {"e_up": P(ep, None, None), "e_down": P(ep, None, None)}

    def layer(ld):
        return {k: col.get(k) or row.get(k) or exp.get(k) or P() for k in ld}

    # same key order as the parameter tree (pytrees flatten dicts in insertion order)
    return {k: ({name: layer(ld) for name, ld in v.items()} if k == "layers" else P()) for k, v in params_like.items()}


def state_specs(cfg: tf.ModelConfig, state_like: dict) -> dict:
    ps = param_specs(cfg, state_like["params"])
    return {k: (jp.PartitionSpec() if k == "step" else ps) for k in state_like}
