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
``mark_stage_end`` after the last block of every stage (``ModelConfig.stage_sizes``; equal stages by default).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any

import torch

from ..ops import core as ops
from ..parallel import tp as tpops
from ..pipelining import mark_stage_end


# parameters of a block that its attention half uses; the others belong to the feed-forward half
ATTN_HALF_KEYS = frozenset({"attn_norm", "wqkv", "wo", "b_qkv", "b_o", "ln1_w", "ln1_b"})


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
    # size of every pipeline stage in blocks (``n_stages`` entries that sum to ``n_layers``; None = equal stages).  An
    # entry may end in .5: a block is two halves, the attention half (norm, qkv, attention, output projection, residual)
    # and the feed-forward half, and a stage boundary may fall between them.  The first stage also embeds the tokens and
    # the last one carries the final norm, the output projection and the cross entropy, so equal block counts leave
    # the rank that holds the last stage busier than the rest; ``balanced_stage_layers`` picks sizes that even out
    # the pipeline ranks' total work.
    stage_layers: tuple | None = None

    def __post_init__(self):
        if self.stage_layers is not None:
            sl = tuple(float(n) for n in self.stage_layers)
            if (len(sl) != self.n_stages or abs(sum(sl) - self.n_layers) > 1e-9 or min(sl) < 0.5
                    or any(abs(2 * n - round(2 * n)) > 1e-9 for n in sl)):
                raise ValueError(f"stage_layers {sl} must have n_stages={self.n_stages} entries that are multiples of 0.5, "
                                 f"at least 0.5 each, and sum to n_layers={self.n_layers}")
            object.__setattr__(self, "stage_layers", tuple(int(n) if n == int(n) else n for n in sl))

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @property
    def layers_per_stage(self) -> int:
        """Blocks per stage when the stages are equal (see ``stage_sizes`` for the general case)."""
        if self.stage_layers is not None and len(set(self.stage_layers)) > 1:
            raise ValueError("stages have different sizes: use stage_sizes / stage_of_half")
        assert self.n_layers % self.n_stages == 0
        return self.n_layers // self.n_stages

    @property
    def stage_sizes(self) -> tuple:
        if self.stage_layers is not None:
            return self.stage_layers
        assert self.n_layers % self.n_stages == 0, "n_layers must be a multiple of n_stages (or give stage_layers)"
        return (self.n_layers // self.n_stages,) * self.n_stages

    @property
    def stage_ends_half(self) -> tuple:
        """For every stage, one past its last half-block (half-block 2*i is the attention half of block i,
        2*i + 1 its feed-forward half)."""
        out, acc = [], 0
        for n in self.stage_sizes:
            acc += int(round(2 * n))
            out.append(acc)
        return tuple(out)

    def stage_of_half(self, half: int) -> int:
        for s, end in enumerate(self.stage_ends_half):
            if half < end:
                return s
        raise IndexError(half)

    def stage_of_layer(self, layer: int) -> int:
        """Stage of a block that is not cut by a stage boundary (of its attention half otherwise)."""
        return self.stage_of_half(2 * layer)

    def stage_of_param(self, layer: int, key: str) -> int:
        """Stage that uses parameter ``key`` of block ``layer``."""
        return self.stage_of_half(2 * layer + (0 if key in ATTN_HALF_KEYS else 1))

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


def stage_cost_model(cfg: "ModelConfig") -> tuple:
    """``(attn_share, head_extra, first_extra)`` for :func:`balanced_stage_layers`, from training FLOPs per token: the
    share of a block's time spent in its attention half, and the cost, in blocks, of the extra work of the output stage
    (final norm, output projection, cross entropy) and of the first stage.  Attention-kernel FLOPs count twice (the
    flash-attention kernels run at about half the rate of the GEMMs, per the per-op timings of a step) and the output
    projection gets 12 % on top for the cross entropy's passes over the logits.  The per-op timings of a step on 8 GPUs
    agree with this within what they can resolve (output projection + loss: 5.1 ms against 11.5 ms for a block, forward
    and backward, i.e. 0.44; the first stage's embedding is below 0.05): the per-TASK times do not, because a task's
    first kernel waits on the stream for the activation from the previous rank, which makes forward tasks of later
    ranks look longer than their work."""
    d, hd = cfg.d_model, cfg.head_dim
    attn_w = d * (cfg.n_heads + 2 * cfg.n_kv_heads) * hd + cfg.n_heads * hd * d
    mlp_w = (3 if cfg.family in ("llama", "mixtral") else 2) * d * cfg.ffn * (cfg.top_k if cfg.n_experts else 1)
    attn_kernels = 2.0 * 3.5 * 4.0 * cfg.seq * cfg.n_heads * hd * (0.5 if cfg.causal else 1.0)
    attn_half = 6.0 * attn_w + attn_kernels
    block = attn_half + 6.0 * mlp_w
    head = 6.0 * cfg.padded_vocab * d * 1.12 if cfg.family != "encoder" else 0.0
    return attn_half / block, head / block, 0.0


def launch_bound(cfg: "ModelConfig", tokens_per_microbatch: int) -> bool:
    """Is a block's GPU time below the time Python needs to launch its kernels?  A block is about 110 launches forward
    and backward at 25-35 us of host time each (measured: 33 us per launch on a step of the GPT-2-XL shape with one
    sequence per replica, where the GPUs ran at 0.11 of the GEMM peak and full clock); its GPU time is estimated from
    its FLOPs at 1e15 FLOP/s.  In such a configuration a stage's cost is its NUMBER of kernels, not their work: the
    output stage's extra is a dozen launches, not the FLOPs of the output projection."""
    d, hd = cfg.d_model, cfg.head_dim
    attn_w = d * (cfg.n_heads + 2 * cfg.n_kv_heads) * hd + cfg.n_heads * hd * d
    mlp_w = (3 if cfg.family in ("llama", "mixtral") else 2) * d * cfg.ffn * (cfg.top_k if cfg.n_experts else 1)
    gpu_ms = 6.0 * (attn_w + mlp_w) * tokens_per_microbatch / max(1, cfg.tp) / 1e15 * 1e3
    host_ms = 110 * 0.030
    return gpu_ms < host_ms


def rank_loads(sizes, stage_to_rank, n_ranks: int, attn_share: float, first_extra: float, last_extra: float) -> list:
    """Work per pipeline rank, in blocks, of stages of ``sizes`` blocks (entries may end in .5) placed by
    ``stage_to_rank``.  The attention half of a block costs ``attn_share`` of a block; the first stage carries
    ``first_extra`` and the last one ``last_extra`` blocks' worth of other work."""
    loads = [0.0] * n_ranks
    half = 0
    for s, n in enumerate(sizes):
        cost = 0.0
        for _ in range(int(round(2 * n))):
            cost += attn_share if half % 2 == 0 else 1.0 - attn_share
            half += 1
        if s == 0:
            cost += first_extra
        if s == len(sizes) - 1:
            cost += last_extra
        loads[stage_to_rank(s)] += cost
    return loads


def balanced_stage_layers(n_layers: int, n_stages: int, stage_to_rank=None, n_ranks: int | None = None,
                          first_extra: float = 0.0, last_extra: float = 0.0, attn_share: float = 0.36,
                          max_shift: float = 1.0, tolerance: float = 0.05) -> tuple:
    """Stage sizes (blocks, multiples of 0.5) that minimise the work of the busiest pipeline rank -- what paces a
    pipeline in its steady state -- when the first stage carries ``first_extra`` and the last stage ``last_extra``
    blocks' worth of other work (embedding; final norm + output projection + cross entropy).

    ``stage_to_rank`` is the schedule's placement (``schedule.get_mpmd_idx``; default: one stage per rank).  Every
    boundary moves at most ``max_shift`` blocks away from the equal split; among splits whose busiest rank is within
    ``tolerance`` blocks of the best the one closest to equal wins.  With measured task times the extras are
    ``t_head / t_block`` etc.
    """
    if n_layers % n_stages:
        raise ValueError("the equal split needs n_layers to be a multiple of n_stages")
    if stage_to_rank is None:
        stage_to_rank, n_ranks = (lambda s: s), n_stages
    if n_ranks is None:
        n_ranks = max(stage_to_rank(s) for s in range(n_stages)) + 1
    per = 2 * (n_layers // n_stages)                      # half-blocks per stage of the equal split
    shifts = range(-int(round(2 * max_shift)), int(round(2 * max_shift)) + 1)
    best = None
    import itertools

    for combo in itertools.product(shifts, repeat=n_stages - 1):
        cuts = [per * (k + 1) + d for k, d in enumerate(combo)]
        bounds = [0] + cuts + [2 * n_layers]
        if any(b1 - b0 < 1 for b0, b1 in zip(bounds, bounds[1:])):
            continue
        sizes = tuple((b1 - b0) / 2 for b0, b1 in zip(bounds, bounds[1:]))
        loads = rank_loads(sizes, stage_to_rank, n_ranks, attn_share, first_extra, last_extra)
        key = (int(max(loads) / tolerance + 1e-6), sum(abs(d) for d in combo), combo)
        if best is None or key < best[0]:
            best = (key, sizes)
    return tuple(int(n) if n == int(n) else n for n in best[1])


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


# Every block is two halves with the residual stream as their only link, so that a pipeline stage boundary can fall
# between them: ``<family>_attn(cfg, p, x, batch, rope) -> x`` and ``<family>_ffn(cfg, p, x) -> x`` (mixtral: (x, aux)).
def llama_attn(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    h = ops.rmsnorm(x, p["attn_norm"], cfg.eps)[0]
    qkv = tpops.column_linear(h, p["wqkv"], None, cfg)
    a = _attention(cfg, qkv, batch, rope)
    return x + tpops.row_linear(a, p["wo"], None, cfg)


def llama_ffn(cfg: ModelConfig, p: dict, x: torch.Tensor) -> torch.Tensor:
    h = ops.rmsnorm(x, p["ffn_norm"], cfg.eps)[0]
    gu = tpops.column_linear(h, p["w_up"], None, cfg)
    return x + tpops.row_linear(ops.swiglu(gu), p["w_down"], None, cfg)


def llama_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    return llama_ffn(cfg, p, llama_attn(cfg, p, x, batch, rope))


def mixtral_ffn(cfg: ModelConfig, p: dict, x: torch.Tensor):
    from ..parallel import moe

    h = ops.rmsnorm(x, p["ffn_norm"], cfg.eps)[0]
    y, aux = moe.moe_ffn(h, {"router": p["router"], "w_up": p["e_up"], "w_down": p["e_down"]}, cfg.n_experts, cfg.top_k,
                         cfg.capacity_factor, cfg.ep, cfg.ep_axis)
    return x + y, aux


def mixtral_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope):
    """Llama attention + top-k mixture-of-experts SwiGLU FFN; returns (x, load-balancing loss of this block)."""
    return mixtral_ffn(cfg, p, llama_attn(cfg, p, x, batch, rope))


def gpt2_attn(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    h = ops.layernorm(x, p["ln1_w"], p["ln1_b"], cfg.eps)[0]
    qkv = tpops.column_linear(h, p["wqkv"], p["b_qkv"], cfg)
    a = _attention(cfg, qkv, batch, None)
    return x + tpops.row_linear(a, p["wo"], p["b_o"], cfg)


def gpt2_ffn(cfg: ModelConfig, p: dict, x: torch.Tensor) -> torch.Tensor:
    h = ops.layernorm(x, p["ln2_w"], p["ln2_b"], cfg.eps)[0]
    u = ops.gelu(tpops.column_linear(h, p["w_up"], p["b_up"], cfg))
    return x + tpops.row_linear(u, p["w_down"], p["b_down"], cfg)


def gpt2_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    return gpt2_ffn(cfg, p, gpt2_attn(cfg, p, x, batch, rope))


def encoder_attn(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    qkv = tpops.column_linear(x, p["wqkv"], p["b_qkv"], cfg)
    a = _attention(cfg, qkv, batch, None)
    return ops.layernorm(x + tpops.row_linear(a, p["wo"], p["b_o"], cfg), p["ln1_w"], p["ln1_b"], cfg.eps)[0]


def encoder_ffn(cfg: ModelConfig, p: dict, x: torch.Tensor) -> torch.Tensor:
    u = ops.gelu(tpops.column_linear(x, p["w_up"], p["b_up"], cfg))
    return ops.layernorm(x + tpops.row_linear(u, p["w_down"], p["b_down"], cfg), p["ln2_w"], p["ln2_b"], cfg.eps)[0]


def encoder_block(cfg: ModelConfig, p: dict, x: torch.Tensor, batch: int, rope) -> torch.Tensor:
    """Post-LayerNorm block: x = LN(x + Attn(x)); x = LN(x + FFN(x))."""
    return encoder_ffn(cfg, p, encoder_attn(cfg, p, x, batch, rope))


_BLOCKS = {"llama": llama_block, "gpt2": gpt2_block, "encoder": encoder_block, "mixtral": mixtral_block}
_HALVES = {"llama": (llama_attn, llama_ffn), "gpt2": (gpt2_attn, gpt2_ffn), "encoder": (encoder_attn, encoder_ffn),
           "mixtral": (llama_attn, mixtral_ffn)}


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


def run_layers(cfg: ModelConfig, params: dict, x: torch.Tensor, batch: int, rope=None):
    """Apply every block in ``params['layers']`` with a stage marker at the end of every stage but the final one
    (whose marker follows the loss).  A stage may end between the two halves of a block (``ModelConfig.stage_layers``);
    such a block runs (and, with ``recompute``, is recomputed) as two halves, every other block as one unit.
    Returns ``x``, or ``(x, aux)`` for the mixture-of-experts family."""
    cuts = set(cfg.stage_ends_half[:-1])
    moe_family = cfg.family == "mixtral"
    aux = torch.zeros((), dtype=torch.float32, device=x.device) if moe_family else None
    block = _BLOCKS[cfg.family]
    attn_half, ffn_half = _HALVES[cfg.family]

    def mark(x_, aux_):
        if moe_family:
            return mark_stage_end((x_, aux_))
        return mark_stage_end(x_), aux_

    for name in sorted(params["layers"]):
        i = int(name)
        p = params["layers"][name]
        if 2 * i + 1 in cuts:     # a stage ends after this block's attention half
            x = _maybe_recompute(cfg, attn_half, {k: v for k, v in p.items() if k in ATTN_HALF_KEYS}, x, batch, rope)
            x, aux = mark(x, aux)
            out = _maybe_recompute(cfg, lambda c, q, x_, b_, r_: ffn_half(c, q, x_),
                                   {k: v for k, v in p.items() if k not in ATTN_HALF_KEYS}, x, batch, None)
        else:
            out = _maybe_recompute(cfg, block, p, x, batch, rope)
        if moe_family:
            x, a = out
            aux = aux + a
        else:
            x = out
        if 2 * i + 2 in cuts:
            x, aux = mark(x, aux)
    return (x, aux) if moe_family else x


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
