"""MpmdArray / MpmdSharding semantics and SPMD<->MPMD resharding on a single-process multi-device CPU mesh
(the behaviours of the reference's tests/test_mpmd_array.py:14-117 and tests/test_reshard_utils.py:29-233)."""
import pytest
import torch

import jaxpp_b200 as jp
from jaxpp_b200.array import DistArray, MpmdArray, MpmdSharding, mpmd_to_spmd_reshard, plan_reshard, spmd_to_mpmd_reshard
from jaxpp_b200.mesh import NamedSharding

P = jp.PartitionSpec


def mesh_3x2():
    return jp.MpmdMesh.create({"mpmd": 3, "data": 2, "model": 1}, kind="cpu", multi_process=False)


def local_array(mesh, idx, x, spec):
    return DistArray.from_global(x, NamedSharding(mesh.unstack[idx], spec))


def test_replicated_and_single_rank_arrays():
    mesh = mesh_3x2()
    x = torch.arange(24.0).reshape(4, 6)
    spec = P("data", None)
    single = MpmdArray([local_array(mesh, 1, x, spec)], MpmdSharding(mesh, {1}, spec))
    assert single.mpmd_idxs == (1,) and not single.is_mpmd_replicated and single.is_partially_addressable
    assert single.shape == (4, 6) and single.dtype == torch.float32 and single.ndim == 2 and single.spec == spec
    torch.testing.assert_close(single.to_mpmd_local_array.to_global(), x)
    assert single.first_mpmd_replica is single.to_mpmd_local_array

    rep = MpmdArray([local_array(mesh, 0, x, spec), local_array(mesh, 2, x, spec)], MpmdSharding(mesh, {0, 2}, spec))
    assert rep.mpmd_idxs == (0, 2) and rep.is_mpmd_replicated
    assert isinstance(rep.to_mpmd_local_array, list) and len(rep.to_mpmd_local_array) == 2
    assert rep.first_mpmd_replica is rep.to_mpmd_local_array[0]
    # the union sharding covers the devices of ranks 0 and 2
    assert set(rep.sharding.mesh.flat_devices) == set(mesh.unstack[0].flat_devices) | set(mesh.unstack[2].flat_devices)


def test_metadata_only_array_and_constructor_checks():
    mesh = mesh_3x2()
    spec = P(None)
    meta = MpmdArray([], MpmdSharding(mesh, {2}, spec), shape=(5,), dtype=torch.bfloat16)
    assert not meta.is_partially_addressable and meta.to_mpmd_local_array is None and meta.first_mpmd_replica is None
    assert meta.local_tensor() is None and meta.shape == (5,) and meta.dtype == torch.bfloat16
    with pytest.raises(AssertionError, match="not partially addressable"):
        float(meta)
    x = torch.ones(5)
    with pytest.raises(ValueError, match="not in mpmd_idxs"):
        MpmdArray([local_array(mesh, 0, x, spec)], MpmdSharding(mesh, {1}, spec))
    with pytest.raises(ValueError, match="already has a mpmd_idx"):
        MpmdArray([local_array(mesh, 1, x, spec), local_array(mesh, 1, x, spec)], MpmdSharding(mesh, {1}, spec))
    # the stage axis never shards inside a stage: it is filtered from the spec
    assert MpmdSharding(mesh, {0}, P("mpmd", "data")).spec == P(None, "data")


def test_scalar_formatting_and_delete():
    mesh = mesh_3x2()
    loss = MpmdArray([local_array(mesh, 2, torch.tensor(1.25), P())], MpmdSharding(mesh, {2}, P()))
    assert f"{loss:.3f}" == "1.250" and float(loss) == 1.25 and int(loss) == 1
    assert not loss.is_deleted()
    loss.delete()
    assert loss.is_deleted()
    with pytest.raises(AssertionError, match="deleted"):
        loss.to_mpmd_local_array


SPECS = [P(), P("data"), P(None, "data"), P(("mpmd", "data")), P("mpmd", "data"), P("data", "mpmd")]


@pytest.mark.parametrize("spmd_spec", SPECS)
@pytest.mark.parametrize("mpmd_spec", [P(), P("data"), P(None, "data")])
def test_spmd_to_mpmd_and_back(spmd_spec, mpmd_spec):
    """Arrays sharded over the whole mesh (specs may mention the stage axis) move to the ranks that use them and
    back; values survive, placement follows the MpmdSharding."""
    mesh = mesh_3x2()
    full = NamedSharding(mesh.jax_mesh, spmd_spec)
    xs = [torch.arange(72.0).reshape(12, 6) + 100 * i for i in range(3)]
    arrays = [DistArray.from_global(x, full) for x in xs]
    targets = [MpmdSharding(mesh, {0}, mpmd_spec), MpmdSharding(mesh, {1, 2}, mpmd_spec), MpmdSharding(mesh, set(), mpmd_spec)]
    moved = spmd_to_mpmd_reshard(mesh, arrays, targets, threshold=1, donate=False)   # threshold 1: one array per group
    assert [m.mpmd_idxs for m in moved] == [(0,), (1, 2), (0,)]                      # unused inputs are parked on rank 0
    for m, x in zip(moved, xs):
        locs = m.to_mpmd_local_array
        for arr in (locs if isinstance(locs, list) else [locs]):
            torch.testing.assert_close(arr.to_global(), x)
            assert arr.spec == m.spec
    back = mpmd_to_spmd_reshard(mesh, moved, [full] * 3)
    for b, x in zip(back, xs):
        assert b.sharding == full
        torch.testing.assert_close(b.to_global(), x)


def test_reshard_plan_between_different_mesh_shapes():
    """Source and destination meshes of different shapes over the same devices: the plan is a set of box copies that
    covers every destination shard exactly once."""
    a = jp.MpmdMesh.create({"mpmd": 1, "data": 4, "model": 1}, kind="cpu", multi_process=False)
    b = jp.MpmdMesh.create({"mpmd": 1, "data": 2, "model": 2}, kind="cpu", multi_process=False)
    src, dst = NamedSharding(a.jax_mesh, P("data", None)), NamedSharding(b.jax_mesh, P("model", "data"))
    ops = plan_reshard((8, 6), src, dst)
    covered = {}
    for op in ops:
        covered[op.dst] = covered.get(op.dst, 0) + op.numel
    assert set(covered) == set(b.jax_mesh.flat_devices) and all(v == 4 * 3 for v in covered.values())
    x = torch.arange(48.0).reshape(8, 6)
    from jaxpp_b200.array import reshard

    torch.testing.assert_close(reshard(DistArray.from_global(x, src), dst).to_global(), x)


def test_logically_stacked_view_over_the_whole_mesh():
    """Per-rank copies of an array seen as one array with a leading stage dimension split over the stage axis
    (reference: array.py:553-600): no data moves, the global view stacks the ranks' values."""
    from jaxpp_b200.array import logically_stacked

    mesh = mesh_3x2()
    xs = [torch.arange(24.0).reshape(4, 6) + 100 * i for i in range(3)]
    whole = mesh.jax_mesh
    shards = {}
    for i in range(3):
        shards.update(local_array(mesh, i, xs[i], P("data", None)).shards)
    per_rank = DistArray(shards, NamedSharding(mesh.unstack[0], P("data", None)), (4, 6))
    stacked = logically_stacked(per_rank, whole, "mpmd")
    assert stacked.shape == (3, 4, 6) and stacked.spec == P("mpmd", "data", None)
    torch.testing.assert_close(stacked.to_global(), torch.stack(xs))
    for d, t in stacked.shards.items():
        assert t.data_ptr() == shards[d].data_ptr()        # a view: nothing was copied
    inner = logically_stacked(per_rank, whole, "mpmd", array_axis=1)
    assert inner.shape == (4, 3, 6) and inner.spec == P("data", "mpmd", None)
    torch.testing.assert_close(inner.to_global(), torch.stack(xs, dim=1))
    with pytest.raises(AssertionError, match="already exists"):
        logically_stacked(DistArray(shards, NamedSharding(whole, P("mpmd", None)), (6, 6)), whole, "mpmd", strict=True)
