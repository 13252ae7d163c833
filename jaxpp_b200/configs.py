"""Named run configurations: model shape x mesh x schedule x batch, including the benchmark configurations.

Every configuration maps a GPU count to a mesh ``(mpmd, data, model)``, a schedule and a microbatching; the
batch sizes are *global* (sequences per step over all data-parallel replicas).
"""
from __future__ import annotations

import dataclasses
from typing import Callable

import torch

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
    RunConfig("mixtral8x7b_pp2ep4", tf.mixtral_8x7b, 2, 4, 1, 4, _dpv, 64, 8, ep=4,
              description="Mixtral-8x7B shape, PP2 x EP4 (experts over the data axis), DualPipeV, microbatches of 2 per replica"),
    RunConfig("llama70b_pp4tp2", tf.llama2_70b, 4, 1, 2, 4, _zb, 64, 1, recompute=True,
              description="Llama-2-70B shape, PP4 x TP2, ZeroBubble, 64 microbatches of 1, full activation recompute"),
]}


def get(name: str) -> RunConfig:
    if name not in CONFIGS:
        raise KeyError(f"unknown configuration {name!r}; available: {sorted(CONFIGS)}")
    return CONFIGS[name]
