"""Shared test fixtures: a small MLP/encoder train step and comparison helpers."""
import torch
from torch.utils import _pytree as pytree

import jaxpp_b200 as jp
from jaxpp_b200.ops import core as ops


def mlp_params(n_layers, hidden, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return [
        {
            "w1": (torch.randn(2 * hidden, hidden, generator=g) * 0.2).to(dtype),
            "b1": torch.zeros(2 * hidden, dtype=dtype),
            "w2": (torch.randn(hidden, 2 * hidden, generator=g) * 0.2).to(dtype),
            "g": torch.ones(hidden, dtype=dtype),
            "b": torch.zeros(hidden, dtype=dtype),
        }
        for _ in range(n_layers)
    ]


def mlp_forward(params, x, n_stages):
    per = len(params) // n_stages
    for i, p in enumerate(params):
        h = ops.gelu(ops.linear(x, p["w1"], p["b1"]))
        h = ops.linear(h, p["w2"], None)
        x = ops.layernorm(x + h, p["g"], p["b"], 1e-5)[0]
        if (i + 1) % per == 0:
            x = jp.mark_stage_end(x)
    return x


def make_mlp_step(n_stages, schedule, n_mb, lr=0.1):
    def step(params, batch):
        def body(mb):
            def loss_fn(p):
                out = mlp_forward(p, mb, n_stages)
                return ((out - mb) ** 2).mean() / n_mb

            return jp.value_and_grad(loss_fn)(params)

        loss, grads = jp.treduce(body, batch, schedule=schedule)
        new = pytree.tree_map(lambda p, g: p - lr * g, params, grads)
        return loss, new

    return step


def leaves(tree):
    return pytree.tree_leaves(tree, is_leaf=lambda x: isinstance(x, jp.MpmdArray))


def local(x):
    return x.local_tensor() if isinstance(x, jp.MpmdArray) else x


def assert_trees_equal(ref, got, exact=True, rtol=1e-5, atol=1e-6):
    a, b = leaves(ref), leaves(got)
    assert len(a) == len(b)
    for x, y in zip(a, b):
        y = local(y)
        if exact:
            assert torch.equal(x, y), (x - y).abs().max()
        else:
            torch.testing.assert_close(y, x, rtol=rtol, atol=atol)
