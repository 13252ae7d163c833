"""Checkpoint round trips, including a change of pipeline layout."""
import json
import os

import torch
from torch.utils import _pytree as pytree

import jaxpp_b200 as jp
from jaxpp_b200 import checkpoint as ckpt
from jaxpp_b200.array import DistArray, MpmdArray, MpmdSharding
from jaxpp_b200.mesh import NamedSharding, P

from helpers import make_mlp_step, mlp_params


def mesh_of(pp, tp=1):
    return jp.MpmdMesh.create({"mpmd": pp, "data": 1, "model": tp}, kind="cpu", multi_process=False)


def test_save_load_same_and_different_pipeline_layout(tmp_path):
    sched2 = jp.Std1F1B(2)
    params, batch = mlp_params(4, 8), torch.randn(4, 2, 8)
    step2 = make_mlp_step(2, sched2, 4)
    mesh2 = mesh_of(2)
    f2 = jp.mpmd_jit_with_loop(step2, mesh2)
    loss, new = f2(params, batch)
    count = torch.tensor(3)
    path = ckpt.save(str(tmp_path), 3, {"params": new, "count": count}, mesh2, extra={"cursor": 17, "schedule": "Std1F1B(2)"})
    assert os.path.basename(path) == "step_00000003" and not os.path.exists(path + ".tmp")
    manifest = json.load(open(os.path.join(path, "manifest.json")))
    e = manifest["entries"]["params/0/w1"]
    assert e["shape"] == [16, 8] and e["mesh_ids"] == [0] and len(e["shards"]) == 1
    assert ckpt.latest_step(str(tmp_path)) == 3

    # same layout
    target = {"params": pytree.tree_map(lambda a: a.mpmd_sharding, new, is_leaf=lambda x: isinstance(x, MpmdArray)),
              "count": None}
    got, extra = ckpt.load(str(tmp_path), None, target, mesh2)
    assert extra["cursor"] == 17 and int(got["count"]) == 3
    for a, b in zip(pytree.tree_leaves(new, is_leaf=lambda x: isinstance(x, MpmdArray)),
                    pytree.tree_leaves(got["params"], is_leaf=lambda x: isinstance(x, MpmdArray))):
        assert a.mpmd_idxs == b.mpmd_idxs and torch.equal(a.local_tensor(), b.local_tensor())

    # resume on a 4-rank pipeline: every layer on its own rank
    mesh4 = mesh_of(4)
    target4 = {"params": [{k: MpmdSharding(mesh4, {i}, P()) for k in layer} for i, layer in enumerate(params)],
               "count": None}
    got4, _ = ckpt.load(str(tmp_path), 3, target4, mesh4)
    assert got4["params"][3]["w1"].mpmd_idxs == (3,)
    sched4 = jp.Std1F1B(4)
    f4 = jp.mpmd_jit_with_loop(make_mlp_step(4, sched4, 4), mesh4)
    ref_loss, ref_new = make_mlp_step(4, sched4, 4)(pytree.tree_map(lambda a: a.local_tensor(), new,
                                                                    is_leaf=lambda x: isinstance(x, MpmdArray)), batch)
    loss4, new4 = f4(got4["params"], batch)
    assert torch.equal(loss4.local_tensor(), ref_loss)


def test_sharded_entries_reassemble_across_tensor_parallel_sizes(tmp_path):
    """An array saved as two row shards restores as four column shards (and whole)."""
    mesh = mesh_of(1, tp=2)
    x = torch.arange(64.0).view(8, 8)
    sub = mesh.unstack[0]
    arr = MpmdArray([DistArray.from_global(x, NamedSharding(sub, P("model", None)))], MpmdSharding(mesh, {0}, P("model", None)))
    rep = MpmdArray([DistArray.from_global(x, NamedSharding(sub, P()))], MpmdSharding(mesh, {0}, P()))
    path = ckpt.save(str(tmp_path), 0, {"w": arr, "r": rep}, mesh)
    entries = json.load(open(os.path.join(path, "manifest.json")))["entries"]
    assert len(entries["w"]["shards"]) == 2 and len(entries["r"]["shards"]) == 1  # replicas are written once
    mesh4 = mesh_of(1, tp=4)
    got, _ = ckpt.load(str(tmp_path), 0, {"w": MpmdSharding(mesh4, {0}, P(None, "model")), "r": None}, mesh4)
    local = got["w"].to_mpmd_local_array
    assert local.to_global().equal(x) and torch.equal(got["r"], x)
    d2 = mesh4.unstack[0].flat_devices[2]
    assert torch.equal(local.shards[d2], x[:, 4:6])
