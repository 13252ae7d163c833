"""Transformer model families as pure functions over parameter pytrees.

Three decoder/encoder families cover the benchmark configurations:

* ``encoder`` — BERT-style post-LayerNorm encoder block (GELU FFN), the analogue of the reference's
  example model (examples/basic.py:33-91);
* ``gpt2``    — pre-LayerNorm decoder with learned positions and GELU FFN;
* ``llama``   — pre-RMSNorm decoder with RoPE, SwiGLU FFN and grouped-query attention (Llama-2, and the
  dense part of Mixtral).

Models are written against the local shard a device sees.  With a ``model`` (tensor-parallel) axis of
size ``tp`` the layers follow the Megatron sequence-parallel recipe: activations between blocks are sharded
over tokens, column-parallel linears gather them (``ag_linear``), row-parallel linears reduce-scatter
their output (``linear_rs``); parameters that are replicated across the axis (norm weights, embeddings,
LM head) get their gradients summed with :func:`sync_replicated_grads`.  Stage boundaries are marked with
``mark_stage_end`` every ``layers_per_stage`` layers.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any

import torch

from ..ops import core as ops
from ..parallel import tp as tpops
from ..pipelining import mark_stage_end


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    family: str  # "encoder" | "gpt2" | "llama"
    vocab: int
    d_model: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    ffn: int
    seq: int
    n_stages: int = 1
    tp: int = 1  # size of the tensor-parallel (model) axis
    tp_axis: str = "model"
    eps: float = 1e-5
    rope_theta: float = 10000.0
    dtype: torch.dtype = torch.bfloat16
    causal: bool = True
    tie_embeddings: bool = False
    recompute: bool = False  # recompute each block's activations in backward
    # mixture of experts ("mixtral" family)
    n_experts: int = 0
    top_k: int = 2
    capacity_factor: float = 1.25
    ep: int = 1  # expert-parallel size (experts are sharded over ``ep_axis``; everything else is replicated there)
    ep_axis: str = "data"
    aux_coef: float = 0.01
    # context parallelism: every sequence is split into ``cp`` contiguous chunks over ``cp_axis`` (attention runs as
    # ring attention, everything else is token-local; parameters are replicas over the axis, their gradients are
    # summed over it like data-parallel ones).  ``seq`` stays the full sequence length.  RoPE families only.
    # the output projection split by vocabulary rows over the tensor-parallel axis: logits stay sharded and the cross
    # entropy combines the ranks' log-sum-exps (``tp.vocab_parallel_cross_entropy``); needs untied embeddings
    vocab_parallel: bool = False
    cp: int = 1
    cp_axis: str = "data"
    cp_layout: str = "contiguous"   # or "zigzag": pieces r and 2*cp-1-r per rank, which balances causal attention

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @property
    def layers_per_stage(self) -> int:
        assert self.n_layers % self.n_stages == 0
        return self.n_layers // self.n_stages

    @property
    def padded_vocab(self) -> int:
        return (self.vocab + 127) // 128 * 128

    def n_params(self) -> int:
        d, f = self.d_model, self.ffn
        hd = self.head_dim
        attn = d * (self.n_heads + 2 * self.n_kv_heads) * hd + self.n_heads * hd * d
        mlp = (3 if self.family in ("llama", "mixtral") else 2) * d * f * max(1, self.n_experts)
        emb = self.padded_vocab * d * (1 if self.tie_embeddings or self.family == "encoder" else 2)
        return self.n_layers * (attn + mlp) + emb

    def flops_per_token(self) -> float:
        """Training FLOPs per token: 6 per parameter in a matmul plus causal attention."""
        d, f, hd = self.d_model, self.ffn, self.head_dim
        attn_w = d * (self.n_heads + 2 * self.n_kv_heads) * hd + self.n_heads * hd * d
        mlp_w = (3 if self.family in ("llama", "mixtral") else 2) * d * f * (self.top_k if self.n_experts else 1)
        head = self.padded_vocab * d if self.family != "encoder" else 0
        matmul = 6.0 * (self.n_layers * (attn_w + mlp_w) + head)
        attn = 12.0 * self.n_layers * self.n_heads * hd * self.seq * (0.5 if self.causal else 1.0)
        return matmul + attn


# presets named after the shapes in the benchmark configurations
def llama2_7b(**kw) -> ModelConfig:
    return ModelConfig("llama", 32000, 4096, 32, 32, 32, 11008, 4096, **kw)


def llama2_70b(**kw) -> ModelConfig:
    return ModelConfig("llama", 32000, 8192, 80, 64, 8, 28672, 4096, **kw)


def mixtral_8x7b(**kw) -> ModelConfig:
    return ModelConfig("mixtral", 32000, 4096, 32, 32, 8, 14336, 4096, n_experts=8, top_k=2, **kw)


def gpt2_xl(**kw) -> ModelConfig:
    return ModelConfig("gpt2", 50257, 1600, 48, 25, 25, 6400, 1024, **kw)


def bert_example(**kw) -> ModelConfig:
    kw.setdefault("dtype", torch.float32)
    kw.setdefault("causal", False)
    return ModelConfig("encoder", 0, 256, 4, 4, 4, 1024, 128, **kw)


# =============================================================================================
# parameters
# =============================================================================================
def _randn(gen, shape, std, dtype, device):
    if str(device) == "meta":
        return torch.empty(shape, dtype=dtype, device="meta")
    return (torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device) * std).to(dtype=dtype, device=device)


def init_layer(cfg: ModelConfig, layer: int, device="cpu", seed: int = 0, tp_rank: int = 0, dtype=None) -> dict:
    """Parameters of one block (the ``tp_rank``-th shard of the tensor-parallel ones)."""
    dtype = dtype or cfg.dtype
    d, f, hd, tp = cfg.d_model, cfg.ffn, cfg.head_dim, cfg.tp
    gen_dev = device if str(device).startswith("cuda") else "cpu"
    gen = torch.Generator(device=gen_dev).manual_seed(seed * 100003 + layer * 131 + tp_rank)
    std = 0.02
    out_std = std / math.sqrt(2 * cfg.n_layers)
    qkv_rows = (cfg.n_heads + 2 * cfg.n_kv_heads) * hd // tp
    p = {
        "wqkv": _randn(gen, (qkv_rows, d), std, dtype, device),
        "wo": _randn(gen, (d, cfg.n_heads * hd // tp), out_std, dtype, device),
        "w_down": _randn(gen, (d, f // tp), out_std, dtype, device),
    }
    ones = lambda: torch.ones(d, dtype=dtype, device=device)
    zeros = lambda n=d: torch.zeros(n, dtype=dtype, device=device)
    if cfg.family == "llama":
        p["w_up"] = _randn(gen, (2 * f // tp, d), std, dtype, device)  # [gate | up]
        p["attn_norm"], p["ffn_norm"] = ones(), ones()
    elif cfg.family == "mixtral":
        del p["w_down"]
        e_local = cfg.n_experts // cfg.ep
        p["router"] = _randn(gen, (cfg.n_experts, d), std, dtype, device)
        p["e_up"] = _randn(gen, (e_local, 2 * f, d), std, dtype, device)     # this rank's experts, [gate | up]
        p["e_down"] = _randn(gen, (e_local, d, f), out_std, dtype, device)
        p["attn_norm"], p["ffn_norm"] = ones(), ones()
    else:
        p["w_up"] = _randn(gen, (f // tp, d), std, dtype, device)
        p["b_up"] = zeros(f // tp)
        p["b_qkv"] = zeros(qkv_rows)
        p["b_o"], p["b_down"] = zeros(), zeros()
        p["ln1_w"], p["ln1_b"], p["ln2_w"], p["ln2_b"] = ones(), zeros(), ones(), zeros()
    return p


def init_params(cfg: ModelConfig, device="cpu", seed: int = 0, tp_rank: int = 0, layers=None, with_embed=True,
                with_head=True, dtype=None) -> dict:
    """Full parameter tree, or only the listed ``layers`` / embedding / head (for per-stage placement)."""
    dtype = dtype or cfg.dtype
    layers = range(cfg.n_layers) if layers is None else layers
    gen_dev = device if str(device).startswith("cuda") else "cpu"
    gen = torch.Generator(device=gen_dev).manual_seed(seed * 7919 + 17)
    params: dict[str, Any] = {"layers": {f"{i:03d}": init_layer(cfg, i, device, seed, tp_rank, dtype) for i in layers}}
    d = cfg.d_model
    if cfg.family != "encoder":
        if with_embed:
            params["embed"] = _randn(gen, (cfg.padded_vocab, d), 0.02, dtype, device)
            if cfg.family == "gpt2":
                params["pos"] = _randn(gen, (cfg.seq, d), 0.01, dtype, device)
        if with_head:
            params["final_norm"] = torch.ones(d, dtype=dtype, device=device)
            if cfg.family == "gpt2":
                params["final_norm_b"] = torch.zeros(d, dtype=dtype, device=device)
            if not cfg.tie_embeddings:
                params["lm_head"] = _randn(gen, (cfg.padded_vocab, d), 0.02, dtype, device)
                if cfg.vocab_parallel and cfg.tp > 1:   # this rank's rows of the same matrix
                    rows = cfg.padded_vocab // cfg.tp
                    params["lm_head"] = params["lm_head"][tp_rank * rows:(tp_rank + 1) * rows].contiguous()
    return params


def rope_tables(cfg: ModelConfig, device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    half = cfg.head_dim // 2
    inv = cfg.rope_theta ** (-torch.arange(half, dtype=torch.float32, device=device) / half)
    pos = torch.arange(cfg.seq, dtype=torch.float32, device=device)
    if cfg.cp > 1:   # this rank's chunk of every sequence
        from ..parallel import context

        pos = context.local_sequence_slice(pos, cfg.cp_axis, 0, cfg.cp_layout)
    ang = pos[:, None] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


# =============================================================================================
# blocks (x is [tokens_local, d]; tokens = batch * seq, batch-major)
# =============================================================================================
def _attention(cfg: ModelConfig, qkv: torch.Tensor, batch: int, rope) -> torch.Tensor:
    hd, tp = cfg.head_dim, cfg.tp
    hq, hkv = cfg.n_heads // tp, cfg.n_kv_heads // tp
    qkv = qkv.view(batch, -1, hq + 2 * hkv, hd)
    cos, sin = rope if rope is not None else (None, None)
    q, k, v = ops.qkv_split(qkv, cos, sin, hq, hkv)  # one pass: split into contiguous q/k/v + RoPE on q, k
    if cfg.cp > 1:
        from ..parallel import context

        o = context.ring_attention(q, k, v, cfg.causal, hd ** -0.5, cfg.cp_axis, cfg.cp_layout)
    else:
        o, _ = ops.attention(q, k, v, cfg.causal, hd ** -0.5)
    return o.view(-1, hq * hd)


def llama_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    h = ops.rmsnorm(x, p["attn_norm"], cfg.eps)[0]
    qkv = tpops.column_linear(h, p["wqkv"], None, cfg)
    a = _attention(cfg, qkv, batch, rope)
    x = x + tpops.row_linear(a, p["wo"], None, cfg)
    h = ops.rmsnorm(x, p["ffn_norm"], cfg.eps)[0]
    gu = tpops.column_linear(h, p["w_up"], None, cfg)
    x = x + tpops.row_linear(ops.swiglu(gu), p["w_down"], None, cfg)
    return x


def mixtral_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope):
    """Llama attention + top-k mixture-of-experts SwiGLU FFN; returns (x, load-balancing loss of this block)."""
    from ..parallel import moe

    h = ops.rmsnorm(x, p["attn_norm"], cfg.eps)[0]
    qkv = tpops.column_linear(h, p["wqkv"], None, cfg)
    a = _attention(cfg, qkv, batch, rope)
    x = x + tpops.row_linear(a, p["wo"], None, cfg)
    h = ops.rmsnorm(x, p["ffn_norm"], cfg.eps)[0]
    y, aux = moe.moe_ffn(h, {"router": p["router"], "w_up": p["e_up"], "w_down": p["e_down"]}, cfg.n_experts, cfg.top_k,
                         cfg.capacity_factor, cfg.ep, cfg.ep_axis)
    return x + y, aux


def gpt2_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    h = ops.layernorm(x, p["ln1_w"], p["ln1_b"], cfg.eps)[0]
    qkv = tpops.column_linear(h, p["wqkv"], p["b_qkv"], cfg)
    a = _attention(cfg, qkv, batch, None)
    x = x + tpops.row_linear(a, p["wo"], p["b_o"], cfg)
    h = ops.layernorm(x, p["ln2_w"], p["ln2_b"], cfg.eps)[0]
    u = ops.gelu(tpops.column_linear(h, p["w_up"], p["b_up"], cfg))
    x = x + tpops.row_linear(u, p["w_down"], p["b_down"], cfg)
    return x


def encoder_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    """Post-LayerNorm block: x = LN(x + Attn(x)); x = LN(x + FFN(x))."""
    qkv = tpops.column_linear(x, p["wqkv"], p["b_qkv"], cfg)
    a = _attention(cfg, qkv, batch, None)
    x = ops.layernorm(x + tpops.row_linear(a, p["wo"], p["b_o"], cfg), p["ln1_w"], p["ln1_b"], cfg.eps)[0]
    u = ops.gelu(tpops.column_linear(x, p["w_up"], p["b_up"], cfg))
    x = ops.layernorm(x + tpops.row_linear(u, p["w_down"], p["b_down"], cfg), p["ln2_w"], p["ln2_b"], cfg.eps)[0]
    return x


_BLOCKS = {"llama": llama_block, "gpt2": gpt2_block, "encoder": encoder_block}


class _Recompute(torch.autograd.Function):
    """Run ``fn`` without keeping its activations; re-run it in backward (full activation recompute of a block).
    Captured steps see the re-run as ordinary ops inside the backward task of the stage."""

    @staticmethod
    def forward(ctx, fn, *args):
        ctx.fn = fn
        with torch.no_grad():
            out = fn(*args)
        ctx.save_for_backward(*[a for a in args if isinstance(a, torch.Tensor)])
        ctx.is_tensor = [isinstance(a, torch.Tensor) for a in args]
        ctx.others = [a for a in args if not isinstance(a, torch.Tensor)]
        return out

    @staticmethod
    def backward(ctx, *gs):
        saved, others = list(ctx.saved_tensors), list(ctx.others)
        args = []
        for is_t in ctx.is_tensor:
            if is_t:
                a = saved.pop(0)
                args.append(a.detach().requires_grad_(a.is_floating_point()))
            else:
                args.append(others.pop(0))
        with torch.enable_grad():
            out = ctx.fn(*args)
            outs = out if isinstance(out, tuple) else (out,)
            pairs = [(o, g) for o, g in zip(outs, gs) if g is not None and o.requires_grad]   # several outputs: x and aux loss
            diff = [a for a in args if isinstance(a, torch.Tensor) and a.requires_grad]
            grads = list(torch.autograd.grad([o for o, _ in pairs], diff, [g for _, g in pairs], allow_unused=True))
        res = [None]
        for a in args:
            res.append(grads.pop(0) if isinstance(a, torch.Tensor) and a.requires_grad else None)
        return tuple(res)


def _maybe_recompute(cfg: ModelConfig, block, p: dict, x: torch.Tensor, batch: int, rope):
    if not cfg.recompute:
        return block(cfg, p, x, batch, rope)
    keys = sorted(p)
    rope_t = list(rope) if rope is not None else []

    def fn(x_, *flat):
        params = dict(zip(keys, flat[:len(keys)]))
        r = tuple(flat[len(keys):]) if rope is not None else None
        return block(cfg, params, x_, batch, r)

    return _Recompute.apply(fn, x, *[p[k] for k in keys], *rope_t)


def run_layers(cfg: ModelConfig, params: dict, x: torch.Tensor, batch: int, rope=None) -> torch.Tensor:
    """Apply every block in ``params['layers']`` with a stage marker after each ``layers_per_stage``."""
    per = cfg.layers_per_stage
    if cfg.family == "mixtral":
        aux = torch.zeros((), dtype=torch.float32, device=x.device)
        for name in sorted(params["layers"]):
            i = int(name)
            x, a = _maybe_recompute(cfg, mixtral_block, params["layers"][name], x, batch, rope)
            aux = aux + a
            if (i + 1) % per == 0 and (i + 1) < cfg.n_layers:
                x, aux = mark_stage_end((x, aux))
        return x, aux
    block = _BLOCKS[cfg.family]
    for name in sorted(params["layers"]):
        i = int(name)
        x = _maybe_recompute(cfg, block, params["layers"][name], x, batch, rope)
        if (i + 1) % per == 0 and (i + 1) < cfg.n_layers:
            x = mark_stage_end(x)
    return x


def encoder_forward(cfg: ModelConfig, params: dict, hidden: torch.Tensor) -> torch.Tensor:
    """hidden: [batch, seq, d] → same shape; the last stage marker is placed by the caller after the loss
    inputs are formed (a marker is required after the last stage)."""
    b = hidden.shape[0]
    x = run_layers(cfg, params, hidden.reshape(-1, cfg.d_model), b)
    return mark_stage_end(x).view_as(hidden)


def lm_loss(cfg: ModelConfig, params: dict, tokens: torch.Tensor, labels: torch.Tensor, rope=None) -> torch.Tensor:
    """Sum over this device's tokens of the next-token cross entropy.  ``tokens``/``labels`` are
    [batch, seq] int64; with tensor parallelism each device embeds and scores its own slice of the tokens
    (sequence parallel), so the returned value is a partial sum."""
    b = tokens.shape[0]
    tp = cfg.tp
    if cfg.cp > 1 and cfg.family == "gpt2":
        raise NotImplementedError("context parallelism needs rotary positions (learned absolute positions are not split)")
    flat_tok, flat_lab = tokens.reshape(-1), labels.reshape(-1)
    if tp > 1:
        flat_tok, flat_lab = tpops.local_token_slice(flat_tok, cfg), tpops.local_token_slice(flat_lab, cfg)
    x = ops.embedding(flat_tok, params["embed"])
    if cfg.family == "gpt2":
        pos = params["pos"]
        n_local = flat_tok.shape[0]
        pos_ids = tpops.local_positions(n_local, cfg, tokens.device)
        x = x + ops.embedding(pos_ids, pos)
    x = run_layers(cfg, params, x, b, rope)
    aux = None
    if cfg.family == "mixtral":
        x, aux = x
    if cfg.family == "gpt2":
        x = ops.layernorm(x, params["final_norm"], params["final_norm_b"], cfg.eps)[0]
    else:
        x = ops.rmsnorm(x, params["final_norm"], cfg.eps)[0]
    head = params["embed"] if cfg.tie_embeddings else params["lm_head"]
    if cfg.vocab_parallel and tp > 1:
        if cfg.tie_embeddings:
            raise NotImplementedError("a vocabulary-parallel output projection needs untied embeddings")
        # all tokens x this rank's vocabulary rows (all-gather -> GEMM); the per-token loss is shared by the ranks and
        # every rank keeps the part of its own token slice, so that the ranks' partial sums add up to the total
        logits = tpops.column_linear(x, head, None, cfg)
        every = tpops.vocab_parallel_cross_entropy(logits, labels.reshape(-1), cfg.tp_axis)
        loss = tpops.local_token_slice(every, cfg)
    else:
        logits = ops.linear(x, head, None)
        loss, _ = ops.cross_entropy(logits, flat_lab)
    total = loss.sum()
    if aux is not None:  # the load-balancing term is per token: scale it like the summed cross entropy
        total = total + cfg.aux_coef * aux * flat_lab.shape[0]
    return mark_stage_end(total)


def sync_replicated_grads(cfg: ModelConfig, grads: dict) -> dict:
    """Sum over the tensor-parallel axis the gradients of parameters that are replicated across it."""
    if cfg.tp == 1:
        return grads
    rep_layer = {"attn_norm", "ffn_norm", "ln1_w", "ln1_b", "ln2_w", "ln2_b", "b_o", "b_down", "router"}
    out = dict(grads)
    out["layers"] = {
        name: {k: (tpops.all_reduce(g, cfg.tp_axis) if k in rep_layer else g) for k, g in layer.items()}
        for name, layer in grads["layers"].items()
    }
    for k in ("embed", "pos", "final_norm", "final_norm_b", "lm_head"):
        if k == "lm_head" and cfg.vocab_parallel:
            continue   # sharded by vocabulary rows: every rank owns its gradient
        if k in grads:
            out[k] = tpops.all_reduce(grads[k], cfg.tp_axis)
    return out


def sync_data_parallel_grads(cfg: ModelConfig, grads: dict, axis: str) -> dict:
    """Sum gradients over the data-parallel axis.  Expert weights sharded over that axis (``e_up``/``e_down``)
    are owned by one rank each and are left alone."""
    sharded = {"e_up", "e_down"} if cfg.ep > 1 and cfg.ep_axis == axis else set()
    out = dict(grads)
    out["layers"] = {
        name: {k: (g if k in sharded else tpops.all_reduce(g, axis)) for k, g in layer.items()}
        for name, layer in grads["layers"].items()
    }
    for k, g in grads.items():
        if k != "layers":
            out[k] = tpops.all_reduce(g, axis)
    return out


# =============================================================================================
# tensor-parallel sharding of a full (tp = 1) parameter tree
# =============================================================================================
def shard_layer_for_tp(cfg: ModelConfig, full: dict, tp: int, r: int) -> dict:
    """The ``r``-th of ``tp`` shards of one block's parameters.  Column-parallel weights (``wqkv``,
    ``w_up``) are split by output rows — per q/k/v section and per gate/up half so that every shard keeps
    whole heads and matching gate/up columns — row-parallel ones (``wo``, ``w_down``) by input columns;
    everything else is replicated."""
    hd = cfg.head_dim
    hq, hkv = cfg.n_heads * hd, cfg.n_kv_heads * hd
    out = {}

    def rows(t, sections):
        parts, start = [], 0
        for n in sections:
            k = n // tp
            parts.append(t[start + r * k:start + (r + 1) * k])
            start += n
        return torch.cat(parts, 0).contiguous()

    for k, t in full.items():
        if k in ("wqkv", "b_qkv"):
            out[k] = rows(t, (hq, hkv, hkv))
        elif k in ("w_up", "b_up"):
            out[k] = rows(t, (cfg.ffn, cfg.ffn) if cfg.family == "llama" else (cfg.ffn,))
        elif k in ("wo", "w_down"):
            n = t.shape[1] // tp
            out[k] = t[:, r * n:(r + 1) * n].contiguous()
        else:
            out[k] = t
    return out


def shard_params_for_tp(cfg: ModelConfig, full: dict, tp: int, r: int) -> dict:
    out = {k: v for k, v in full.items() if k != "layers"}
    if cfg.vocab_parallel and "lm_head" in out and not isinstance(out["lm_head"], type(None)) and tp > 1:
        rows = out["lm_head"].shape[0] // tp
        out["lm_head"] = out["lm_head"][r * rows:(r + 1) * rows]
    out["layers"] = {name: shard_layer_for_tp(cfg, layer, tp, r) for name, layer in full["layers"].items()}
    return out
