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
from ..parallel import zero
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
    # master weights and Adam moments sharded over the data-parallel ranks (``parallel/zero.py``): the state then
    # holds flat 1/dp slices (``shard_state_for_dp``), gradients are reduce-scattered and parameters all-gathered
    shard_optimizer: bool = False
    # clip the gradient to this global L2 norm (over every pipeline stage, tensor- / expert-parallel shard); None = off
    clip_grad_norm: float | None = None


def stage_of_layer(cfg: tf.ModelConfig, layer: int) -> int:
    return cfg.stage_of_layer(layer)


def owner_ranks(cfg: tf.ModelConfig, schedule) -> dict:
    """Pipeline rank of every parameter group: ``{"embed": r, "head": r, layer index: r, (layer index, half): r}`` with half 0 for
    the parameters of a block's attention half and 1 for those of its feed-forward half (a stage boundary may fall
    between the two, ``ModelConfig.stage_layers``); ``owner_of(owners, layer, key)`` looks a parameter up."""
    out: dict[Any, int] = {}
    for i in range(cfg.n_layers):
        out[i] = int(schedule.get_mpmd_idx(cfg.stage_of_layer(i)))   # a whole block (its attention half when cut)
        for half in (0, 1):
            out[(i, half)] = int(schedule.get_mpmd_idx(cfg.stage_of_half(2 * i + half)))
    out["embed"] = int(schedule.get_mpmd_idx(0))
    out["head"] = int(schedule.get_mpmd_idx(cfg.n_stages - 1))
    return out


def owner_of(owners: dict, layer: int, key: str) -> int:
    return owners[(layer, 0 if key in tf.ATTN_HALF_KEYS else 1)]


def init_state(cfg: tf.ModelConfig, schedule, device, my_rank: int | None = None, tp_rank: int = 0, seed: int = 0) -> dict:
    """Training state for pipeline rank ``my_rank`` (``None`` = everything, for single-process runs).

    Parameter groups owned by other ranks are present as :class:`ShapeDtypeStruct` leaves so that the
    pytree has the same structure on every process.
    """
    owners = owner_ranks(cfg, schedule)
    mine = lambda key: my_rank is None or owners[key] == my_rank
    tied_extra = cfg.tie_embeddings and my_rank is not None and owners["head"] == my_rank
    full = tf.init_params(cfg, "meta", seed, tp_rank)  # structure and shapes only
    local_layers = [i for i in range(cfg.n_layers) if mine((i, 0)) or mine((i, 1))]
    real = tf.init_params(cfg, device, seed, tp_rank, layers=local_layers, with_embed=mine("embed") or tied_extra,
                          with_head=mine("head"))
    for name, layer in real["layers"].items():   # a block cut by a stage boundary: keep the half this rank runs
        for k in [k for k in layer if not mine((int(name), 0 if k in tf.ATTN_HALF_KEYS else 1))]:
            del layer[k]

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

    if cfg.cp > 1:
        # chunks of a sequence over the context axis: parameters are replicas there, so their gradients are summed over
        # it exactly as over a data-parallel axis (each rank contributes its tokens)
        if dp > 1 and dp_axis == cfg.cp_axis:
            raise ValueError(f"axis {dp_axis!r} cannot be the data-parallel and the context-parallel axis at once")
        if dp > 1:
            raise NotImplementedError("context parallelism together with data parallelism needs a mesh axis of its own")
        dp_axis, dp = cfg.cp_axis, cfg.cp

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
        sharded_update = hyper.shard_optimizer and dp_axis is not None and dp > 1
        if dp_axis is not None and dp > 1 and not sharded_update:
            grads = tf.sync_data_parallel_grads(cfg, grads, dp_axis)
        new_step = state["step"] + 1
        whole = _not_replicated_over(cfg, params, dp_axis) if sharded_update else None
        flat_p, spec = pytree.tree_flatten(params)
        flat_g = pytree.tree_leaves(grads)
        keep = pytree.tree_leaves(whole) if sharded_update else [True] * len(flat_p)
        if sharded_update:
            # this rank's slice of the summed gradient (parameters that are not replicas over the axis keep theirs)
            flat_g = [g if k else zero.reduce_scatter_flat(g, dp_axis) for g, k in zip(flat_g, keep)]
        clip = None
        if hyper.clip_grad_norm is not None:
            clip = _clip_coefficient(cfg, schedule, params, flat_g, keep, dp_axis if dp > 1 else None,
                                     hyper.clip_grad_norm, 1.0 / total_tokens)

        def update(p, master, g, m, v, keep_whole=True):
            if clip is not None:
                g = g * clip.to(g.dtype)
            if not keep_whole:
                # AdamW on the slice -> bf16 slice -> parameter gathered from the owners of the slices
                pm, mm, vm, lp = ops.adamw(master, g, m, v, new_step, hyper.lr, hyper.beta1, hyper.beta2, hyper.eps,
                                           hyper.weight_decay if p.dim() > 1 else 0.0, 1.0 / total_tokens, p.dtype,
                                           None, hyper.inplace_update)
                return zero.all_gather_flat(lp, dp_axis, p.numel()).view(p.shape), pm, mm, vm
            pm, mm, vm, lp = ops.adamw(master, g, m, v, new_step, hyper.lr, hyper.beta1, hyper.beta2, hyper.eps,
                                       hyper.weight_decay if p.dim() > 1 else 0.0, 1.0 / total_tokens, p.dtype,
                                       p if hyper.inplace_update else None, hyper.inplace_update)
            return lp, pm, mm, vm

        flat = [update(p, ma, g, m, v, k) for p, ma, g, m, v, k in zip(
            flat_p, pytree.tree_leaves(state["master"]), flat_g, pytree.tree_leaves(state["m"]),
            pytree.tree_leaves(state["v"]), keep)]
        unf = lambda k: pytree.tree_unflatten([f[k] for f in flat], spec)
        new_state = {"params": unf(0), "master": unf(1), "m": unf(2), "v": unf(3), "step": new_step}
        return new_state, losses

    return step


def _clip_coefficient(cfg: tf.ModelConfig, schedule, params: dict, flat_g: list, whole: list, dp_axis: str | None,
                      max_norm: float, grad_scale: float) -> torch.Tensor:
    """min(1, max_norm / ||grad_scale * g||) over the whole model, as a scalar that lives on every pipeline rank.

    Squares are summed per pipeline rank first; parts held as shards are completed over their axis (tensor-parallel
    weights over the model axis, experts over the expert axis, optimizer-state slices over the data axis; replicas
    count once); the per-rank sums meet in one cross-stage all-reduce (what the reference's users do with
    ``cross_mpmd_all_reduce`` for the global gradient norm, api.py:48-54)."""
    owners = owner_ranks(cfg, schedule)
    tp_sharded = {"wqkv", "w_up", "b_qkv", "b_up", "wo", "w_down"} if cfg.tp > 1 else set()
    if cfg.tp > 1 and cfg.vocab_parallel:
        tp_sharded.add("lm_head")
    ep_sharded = {"e_up", "e_down"} if cfg.ep > 1 else set()
    paths = []   # (owner rank, parameter name) in flattening order
    for k, v in params.items():
        if k == "layers":
            for name, ld in v.items():
                paths.extend((owner_of(owners, int(name), kk), kk) for kk in ld)
        else:
            paths.append((owners["embed" if k in ("embed", "pos") else "head"], k))
    assert len(paths) == len(flat_g)
    groups: dict = {}  # (rank, axes to complete over) -> sum of squares
    for (rank, name), g, keep_whole in zip(paths, flat_g, whole):
        axes = []
        if name in tp_sharded:
            axes.append(cfg.tp_axis)
        if name in ep_sharded:
            axes.append(cfg.ep_axis)
        elif not keep_whole:
            axes.append(dp_axis)      # a 1/dp slice of a replicated parameter's gradient
        sq = g.float().pow(2).sum()
        key = (rank, tuple(dict.fromkeys(axes)))
        groups[key] = sq if key not in groups else groups[key] + sq
    per_rank: dict = {}
    for (rank, axes), sq in groups.items():
        for axis in axes:
            sq = tpops.all_reduce(sq.reshape(1), axis).reshape(())
        per_rank[rank] = sq if rank not in per_rank else per_rank[rank] + sq
    parts = [per_rank[r] for r in sorted(per_rank)]
    total = jp.cross_mpmd_all_reduce(*parts) if len(parts) > 1 else parts[0]
    norm = total.sqrt() * grad_scale
    return torch.clamp(max_norm / (norm + 1e-6), max=1.0)


def _not_replicated_over(cfg: tf.ModelConfig, params_like: dict, axis: str | None) -> dict:
    """Tree of booleans shaped like the parameters: True where a parameter is *not* a replica over mesh axis
    ``axis`` (expert weights when the expert-parallel axis is that axis), so its optimizer state stays whole."""
    own = {"e_up", "e_down"} if cfg.ep > 1 and cfg.ep_axis == axis else set()
    return {k: ({name: {kk: kk in own for kk in ld} for name, ld in v.items()} if k == "layers" else False)
            for k, v in params_like.items()}


def shard_state_for_dp(cfg: tf.ModelConfig, state: dict, dp: int, dp_rank: int, dp_axis: str = "data") -> dict:
    """The state that ``Hyper(shard_optimizer=True)`` steps take: ``master`` / ``m`` / ``v`` reduced to data-parallel
    rank ``dp_rank``'s flat slices (parameters that are not replicated over the axis keep their full state)."""
    whole = _not_replicated_over(cfg, state["params"], dp_axis)

    def keep(path):
        node = whole
        for k in path:
            node = node[k] if isinstance(node, dict) else node
        return bool(node)

    return zero.shard_optimizer_state(state, dp, dp_rank, keep)


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
    top = lambda k: P(tp, None) if k == "lm_head" and cfg.vocab_parallel and tp else P()
    return {k: ({name: layer(ld) for name, ld in v.items()} if k == "layers" else top(k)) for k, v in params_like.items()}


def state_specs(cfg: tf.ModelConfig, state_like: dict, shard_optimizer_axis: str | None = None) -> dict:
    """PartitionSpecs of the whole training state.  With ``shard_optimizer_axis`` the optimizer leaves are the flat
    slices of ``shard_state_for_dp``: globally a 1-d array split over that axis."""
    ps = param_specs(cfg, state_like["params"])
    if shard_optimizer_axis is None:
        return {k: (jp.PartitionSpec() if k == "step" else ps) for k in state_like}
    whole = _not_replicated_over(cfg, state_like["params"], shard_optimizer_axis)
    flat = jp.PartitionSpec(shard_optimizer_axis)
    opt = pytree.tree_unflatten(
        [spec if w else flat for spec, w in zip(pytree.tree_leaves(ps, is_leaf=lambda x: isinstance(x, jp.PartitionSpec)),
                                                pytree.tree_leaves(whole))],
        pytree.tree_structure(whole))
    return {k: (jp.PartitionSpec() if k == "step" else ps if k == "params" else opt) for k in state_like}
