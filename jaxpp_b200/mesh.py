"""Device meshes: ``Device``, ``Mesh``, ``PartitionSpec``, ``NamedSharding`` and ``MpmdMesh``.

``MpmdMesh`` has the property surface of the reference's class (src/jaxpp/mesh.py:28-167):
a device mesh with one axis designated as the *mpmd* (pipeline) axis, ``unstack`` into one
sub-mesh per pipeline rank, ``mpmd_submesh``, ``lowering_mesh``, ``my_mpmd_axis_index`` and a
context-manager ``mesh_stack`` through which run-time ops find the active mesh.  There is no
JAX underneath: a :class:`Device` is (global id, owning process, kind) and, in a
one-process-per-GPU launch, device ``i`` is the GPU of ``torch.distributed`` rank ``i``.
``MpmdMesh`` additionally owns the ``torch.distributed`` process groups of every mesh axis
(``axis_group``), which the tensor-/data-/expert-parallel ops use inside a stage.
"""
from __future__ import annotations

import dataclasses
import math
import os
from functools import cached_property
from typing import Any, ClassVar, Iterable, Mapping, Sequence

import numpy as np

from .utils import config


@dataclasses.dataclass(frozen=True, order=True)
class Device:
    id: int
    process_index: int = 0
    kind: str = "cpu"  # "cpu" or "cuda"
    local_index: int = 0  # ordinal within its process / node

    @property
    def torch_device(self):
        import torch

        return torch.device("cuda", self.local_index) if self.kind == "cuda" else torch.device("cpu")

    def __repr__(self) -> str:
        return f"{self.kind}:{self.id}"


class PartitionSpec(tuple):
    """Per-dimension mesh axis names: ``P('data', None, ('model','expert'))``."""

    def __new__(cls, *parts):
        norm = []
        for p in parts:
            if isinstance(p, list):
                p = tuple(p)
            if isinstance(p, tuple) and len(p) == 1:
                p = p[0]
            if isinstance(p, tuple) and len(p) == 0:
                p = None
            norm.append(p)
        return super().__new__(cls, norm)

    def __repr__(self) -> str:
        return "PartitionSpec(" + ", ".join(repr(p) for p in self) + ")"

    def axes_of(self, dim: int) -> tuple[str, ...]:
        if dim >= len(self) or self[dim] is None:
            return ()
        p = self[dim]
        return p if isinstance(p, tuple) else (p,)

    def all_axes(self) -> tuple[str, ...]:
        return tuple(a for d in range(len(self)) for a in self.axes_of(d))


P = PartitionSpec


def filter_axes(spec: PartitionSpec, drop: Iterable[str]) -> PartitionSpec:
    """Spec with the named mesh axes removed (reference: utils.filter_axes)."""
    drop = set(drop)
    out = []
    for d in range(len(spec)):
        kept = tuple(a for a in spec.axes_of(d) if a not in drop)
        out.append(None if not kept else (kept if len(kept) > 1 else kept[0]))
    return PartitionSpec(*out)


def rm_size1_axes(spec: PartitionSpec, mesh: "Mesh") -> PartitionSpec:
    return filter_axes(spec, {a for a in mesh.axis_names if mesh.shape[a] == 1})


class Mesh:
    """An n-d array of devices with named axes."""

    def __init__(self, devices, axis_names: Sequence[str]):
        self.devices = np.asarray(devices, dtype=object)
        self.axis_names = tuple(axis_names)
        if self.devices.ndim != len(self.axis_names):
            raise ValueError(f"{self.devices.ndim}-d device array but axis names {self.axis_names}")

    @property
    def shape(self) -> dict[str, int]:
        return dict(zip(self.axis_names, self.devices.shape))

    @property
    def size(self) -> int:
        return int(self.devices.size)

    @property
    def device_ids(self) -> np.ndarray:
        return np.vectorize(lambda d: d.id, otypes=[np.int64])(self.devices)

    @cached_property
    def flat_devices(self) -> tuple[Device, ...]:
        return tuple(self.devices.flat)

    @cached_property
    def is_multi_process(self) -> bool:
        return len({d.process_index for d in self.flat_devices}) > 1

    @cached_property
    def device_coords(self) -> Mapping[Device, tuple[int, ...]]:
        return {dev: coord for coord, dev in np.ndenumerate(self.devices)}

    def axis_size(self, names) -> int:
        if names is None:
            return 1
        if isinstance(names, str):
            names = (names,)
        return math.prod(self.shape[a] for a in names)

    def __eq__(self, other):
        return (
            isinstance(other, Mesh)
            and self.axis_names == other.axis_names
            and self.devices.shape == other.devices.shape
            and self.flat_devices == other.flat_devices
        )

    def __hash__(self):
        return hash((self.axis_names, self.devices.shape, self.flat_devices))

    def __repr__(self) -> str:
        return f"Mesh({self.shape})"


@dataclasses.dataclass(frozen=True)
class NamedSharding:
    mesh: Mesh
    spec: PartitionSpec

    def shard_shape(self, global_shape: Sequence[int]) -> tuple[int, ...]:
        out = []
        for d, n in enumerate(global_shape):
            k = self.mesh.axis_size(self.spec.axes_of(d))
            if n % k != 0:
                raise ValueError(f"dimension {d} of size {n} is not divisible by {k} ({self.spec})")
            out.append(n // k)
        return tuple(out)

    def device_index(self, device: Device, global_shape: Sequence[int]) -> tuple[slice, ...]:
        """The hyper-rectangle of the global array that ``device`` holds."""
        coord = dict(zip(self.mesh.axis_names, self.mesh.device_coords[device]))
        idx = []
        for d, n in enumerate(global_shape):
            axes = self.spec.axes_of(d)
            k = self.mesh.axis_size(axes)
            pos = 0
            for a in axes:  # major-to-minor over the listed axes
                pos = pos * self.mesh.shape[a] + coord[a]
            step = n // k
            idx.append(slice(pos * step, (pos + 1) * step))
        return tuple(idx)

    def is_fully_replicated(self) -> bool:
        return all(self.mesh.shape[a] == 1 for a in self.spec.all_axes())


def make_devices(n: int, kind: str = "cpu", one_process_per_device: bool = False, devices_per_node: int = 8):
    """``n`` devices; with ``one_process_per_device`` device ``i`` belongs to process ``i``."""
    return [
        Device(i, i if one_process_per_device else 0, kind, (i % devices_per_node) if kind == "cuda" else 0)
        for i in range(n)
    ]


def _current_process_index() -> int:
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:  # pragma: no cover
        pass
    return int(os.environ.get("RANK", "0"))


@dataclasses.dataclass(frozen=True)
class MpmdMesh:
    """A mesh split along ``mpmd_axis_name`` into independent groups (pipeline ranks).

    With shape ``{'mpmd': 4, 'data': 1, 'model': 2}`` there are 4 groups of 2 devices; each
    group runs its own program (MPMD) and is SPMD inside.  In a multi-process launch every
    process must belong to exactly one group (checked at construction, reference :69-84).
    """

    jax_mesh: Mesh  # attribute name kept for API parity; it is a plain :class:`Mesh`
    mpmd_axis_name: str
    mesh_stack: ClassVar[list["MpmdMesh"]] = []

    # -- construction ---------------------------------------------------------------------
    def __post_init__(self):
        if self.mpmd_axis_name not in self.jax_mesh.axis_names:
            raise ValueError(f"{self.mpmd_axis_name!r} is not an axis of {self.jax_mesh}")
        if not self.jax_mesh.is_multi_process:
            return
        seen: dict[int, int] = {}
        for dev in self.jax_mesh.flat_devices:
            idx = self.device_mpmd_idx[dev]
            if seen.setdefault(dev.process_index, idx) != idx:
                raise AssertionError(
                    f"Process {dev.process_index} found in two mpmd indices: {seen[dev.process_index]} {idx}"
                )

    @classmethod
    def create(cls, shape: Mapping[str, int], mpmd_axis_name: str = "mpmd", kind: str | None = None,
               multi_process: bool | None = None) -> "MpmdMesh":
        """Row-major mesh over ``prod(shape)`` devices.

        ``multi_process`` defaults to "torch.distributed is initialised with as many ranks as
        devices"; ``kind`` defaults to cuda when available.
        """
        import torch
        import torch.distributed as dist

        n = math.prod(shape.values())
        if multi_process is None:
            multi_process = dist.is_available() and dist.is_initialized() and dist.get_world_size() == n and n > 1
        if kind is None:
            kind = "cuda" if torch.cuda.is_available() else "cpu"
        per_node = int(os.environ.get("LOCAL_WORLD_SIZE", "8")) if multi_process else max(1, torch.cuda.device_count() or 8)
        devs = make_devices(n, kind, multi_process, per_node)
        mesh = cls(Mesh(np.array(devs, dtype=object).reshape(tuple(shape.values())), tuple(shape.keys())), mpmd_axis_name)
        if multi_process and dist.is_available() and dist.is_initialized() and dist.get_world_size() == n:
            mesh.create_process_groups()  # collectively, while every process is at the same point
        return mesh

    def __enter__(self):
        MpmdMesh.mesh_stack.append(self)
        return self

    def __exit__(self, *exc):
        MpmdMesh.mesh_stack.pop()

    @classmethod
    def current(cls) -> "MpmdMesh":
        if not cls.mesh_stack:
            raise RuntimeError("no MpmdMesh is active; use `with mpmd_mesh:`")
        return cls.mesh_stack[-1]

    # -- geometry ---------------------------------------------------------------------------
    @cached_property
    def device_coords(self) -> Mapping[Device, tuple[int, ...]]:
        return self.jax_mesh.device_coords

    @cached_property
    def mpmd_axis(self) -> int:
        return self.jax_mesh.axis_names.index(self.mpmd_axis_name)

    @cached_property
    def device_mpmd_idx(self) -> Mapping[Device, int]:
        return {d: c[self.mpmd_axis] for d, c in self.device_coords.items()}

    @cached_property
    def mpmd_dim(self) -> int:
        return self.jax_mesh.shape[self.mpmd_axis_name]

    @property
    def axis_names(self) -> tuple[str, ...]:
        return self.jax_mesh.axis_names

    @property
    def shape(self) -> dict[str, int]:
        return self.jax_mesh.shape

    @cached_property
    def unstack(self) -> list[Mesh]:
        parts = np.split(self.jax_mesh.devices, self.mpmd_dim, self.mpmd_axis)
        return [Mesh(p, self.jax_mesh.axis_names) for p in parts]

    @property
    def mpmd_idx_for_mesh(self) -> Mapping[Mesh, int]:
        return {m: i for i, m in enumerate(self.unstack)}

    def mpmd_submesh(self, mpmd_indices: list[int]) -> "MpmdMesh":
        assert isinstance(mpmd_indices, list)
        return MpmdMesh(
            Mesh(np.take(self.jax_mesh.devices, mpmd_indices, self.mpmd_axis), self.jax_mesh.axis_names),
            self.mpmd_axis_name,
        )

    # -- which part is mine -----------------------------------------------------------------
    @cached_property
    def local_devices(self) -> tuple[Device, ...]:
        if not self.jax_mesh.is_multi_process:
            return self.jax_mesh.flat_devices
        me = _current_process_index()
        return tuple(d for d in self.jax_mesh.flat_devices if d.process_index == me)

    @cached_property
    def my_mpmd_axis_index(self) -> int:
        if not config.debug_force_mpmdify.value and not self.jax_mesh.is_multi_process:
            raise ValueError("my_mpmd_axis_index is supported only in multi-process meshes")
        if not self.jax_mesh.is_multi_process:
            return 0
        (idx,) = {self.device_mpmd_idx[d] for d in self.local_devices}
        return idx

    @cached_property
    def my_device(self) -> Device:
        (d,) = self.local_devices
        return d

    @cached_property
    def my_mpmd_group_mesh(self) -> Mesh:
        if not self.jax_mesh.is_multi_process:
            raise ValueError("my_mpmd_group_mesh is supported only in multi-process meshes")
        return self.unstack[self.my_mpmd_axis_index]

    def lowering_mesh(self) -> Mesh:
        """The sub-mesh a stage program is written against: rank 0's slice in one process,
        this process's own slice otherwise."""
        if not self.jax_mesh.is_multi_process:
            return self.unstack[0]
        return self.my_mpmd_group_mesh

    # -- torch.distributed groups -------------------------------------------------------------
    def peers_along(self, axis: str, device: Device | None = None) -> list[Device]:
        """Devices that differ from ``device`` only in their coordinate on ``axis``."""
        device = device or self.my_device
        coord = list(self.device_coords[device])
        ax = self.jax_mesh.axis_names.index(axis)
        out = []
        for i in range(self.jax_mesh.devices.shape[ax]):
            coord[ax] = i
            out.append(self.jax_mesh.devices[tuple(coord)])
        return out

    def axis_index(self, axis: str, device: Device | None = None) -> int:
        device = device or self.my_device
        return self.device_coords[device][self.jax_mesh.axis_names.index(axis)]

    def axis_group(self, axis: str):
        """Process group of this process's peers along ``axis`` (``None`` for size-1 axes or
        single-process meshes).  Groups for *all* lines of the axis are created on first use,
        in the same order on every process, as ``torch.distributed.new_group`` requires."""
        if not self.jax_mesh.is_multi_process or self.jax_mesh.shape[axis] == 1:
            return None
        cache = _GROUP_CACHE.setdefault(self._key(), {})
        if axis not in cache:
            import torch.distributed as dist

            ax = self.jax_mesh.axis_names.index(axis)
            moved = np.moveaxis(self.jax_mesh.devices, ax, -1).reshape(-1, self.jax_mesh.devices.shape[ax])
            mine = None
            for line in moved:
                ranks = [d.process_index for d in line]
                g = dist.new_group(ranks=ranks)
                if self.my_device.process_index in ranks:
                    mine = g
            cache[axis] = mine
        return cache[axis]

    def create_process_groups(self) -> None:
        """Create the process groups of every axis (and of the stages) now.  ``new_group`` is a collective over
        all processes, so creating a group lazily inside a pipeline task would make the ranks of one stage wait
        for ranks of another stage that cannot reach the same point before they receive data: every process
        calls this at the same place instead (mesh creation, start of a multi-controller run)."""
        if not self.jax_mesh.is_multi_process:
            return
        for axis in self.jax_mesh.axis_names:
            self.axis_group(axis)
        self.stage_group()

    def stage_group(self):
        """Process group of all processes in this process's pipeline rank."""
        if not self.jax_mesh.is_multi_process:
            return None
        cache = _GROUP_CACHE.setdefault(self._key(), {})
        if "__stage__" not in cache:
            import torch.distributed as dist

            mine = None
            for sub in self.unstack:
                ranks = [d.process_index for d in sub.flat_devices]
                g = dist.new_group(ranks=ranks) if len(ranks) > 1 else None
                if self.my_device.process_index in ranks:
                    mine = g
            cache["__stage__"] = mine
        return cache["__stage__"]

    def _key(self):
        return (self.jax_mesh.axis_names, self.jax_mesh.devices.shape, tuple(d.id for d in self.jax_mesh.flat_devices))


_GROUP_CACHE: dict[Any, dict[str, Any]] = {}
