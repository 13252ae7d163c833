"""MpmdMesh geometry on a device mesh that needs no hardware."""
import numpy as np
import pytest

from jaxpp_b200.mesh import Mesh, MpmdMesh, NamedSharding, P, filter_axes, make_devices, rm_size1_axes


def test_unstack_16_devices():
    devs = make_devices(16, "cuda")
    mesh = MpmdMesh(Mesh(np.array(devs, dtype=object).reshape(4, 2, 1, 2, 1),
                         ("stage", "data", "sequence", "tensor", "expert")), "stage")
    assert mesh.mpmd_axis == 0 and mesh.mpmd_dim == 4
    assert mesh.device_coords[devs[0]] == (0, 0, 0, 0, 0)
    assert mesh.device_coords[devs[1]] == (0, 0, 0, 1, 0)
    for idx, m in enumerate(mesh.unstack):
        assert m.axis_names == ("stage", "data", "sequence", "tensor", "expert")
        assert m.devices.shape == (1, 2, 1, 2, 1)
        assert (m.device_ids == np.arange(idx * 4, idx * 4 + 4).reshape(1, 2, 1, 2, 1)).all()
    sub = mesh.mpmd_submesh([0, 2])
    assert sub.mpmd_dim == 2 and sub.jax_mesh.device_ids.flatten().tolist() == [0, 1, 2, 3, 8, 9, 10, 11]
    assert mesh.lowering_mesh() == mesh.unstack[0]
    assert mesh.mpmd_idx_for_mesh[mesh.unstack[3]] == 3
    with pytest.raises(ValueError, match="only in multi-process"):
        mesh.my_mpmd_axis_index


def test_process_in_two_groups_rejected():
    devs = make_devices(4, "cuda", one_process_per_device=True)
    devs[2] = type(devs[2])(2, 0, "cuda", 2)  # process 0 owns devices in two pipeline ranks
    with pytest.raises(AssertionError, match="found in two mpmd indices"):
        MpmdMesh(Mesh(np.array(devs, dtype=object).reshape(2, 2), ("mpmd", "model")), "mpmd")


def test_mesh_stack_and_specs():
    mesh = MpmdMesh.create({"mpmd": 2, "data": 1, "model": 2}, kind="cpu", multi_process=False)
    with mesh:
        assert MpmdMesh.current() is mesh
    with pytest.raises(RuntimeError):
        MpmdMesh.current()
    assert filter_axes(P("mpmd", ("data", "model"), None), {"mpmd", "data"}) == P(None, "model", None)
    assert rm_size1_axes(P("data", "model"), mesh.jax_mesh) == P(None, "model")
    sh = NamedSharding(mesh.unstack[1], P(None, "model"))
    assert sh.shard_shape((4, 6)) == (4, 3)
    d = mesh.unstack[1].flat_devices[1]
    assert sh.device_index(d, (4, 6)) == (slice(0, 4), slice(3, 6))
    assert [x.id for x in mesh.peers_along("model", d)] == [2, 3]
