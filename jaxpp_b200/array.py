"""Distributed arrays: ``DistArray`` (SPMD over one mesh), ``MpmdSharding``, ``MpmdArray`` and the
SPMD↔MPMD reshards.

Parity targets in the reference: ``MpmdSharding`` (src/jaxpp/types.py:39-66), ``MpmdArray`` and its
property surface (src/jaxpp/array.py:34-264), ``spmd_to_mpmd_reshard`` with memory-bounded grouping
(:296-541) and ``mpmd_to_spmd_reshard`` (:613-708).  There a reshard is an XLA identity program with
a target sharding; here it is a host-planned set of box copies: every destination shard is the
hyper-rectangle of the global array its device owns, every source shard likewise, and each
non-empty intersection becomes one local copy or one point-to-point message (NCCL/gloo through
``torch.distributed``).
"""
from __future__ import annotations

import dataclasses
import itertools
from collections import OrderedDict
from typing import Any, Iterable, Mapping, Sequence

import torch

from .mesh import Device, Mesh, MpmdMesh, NamedSharding, PartitionSpec, filter_axes, rm_size1_axes
from .utils import hbytes, logger

P = PartitionSpec


# =============================================================================================
# DistArray: one logical array, sharded over the devices of one Mesh
# =============================================================================================
class DistArray:
    """A global array of ``shape`` laid out over ``sharding.mesh`` per ``sharding.spec``.

    ``shards`` maps each *addressable* device to its local tensor (all devices of the mesh in a
    single-process run; this process's device otherwise).
    """

    def __init__(self, shards: Mapping[Device, torch.Tensor], sharding: NamedSharding, shape: Sequence[int],
                 dtype: torch.dtype | None = None):
        self.shards: dict[Device, torch.Tensor | None] = dict(shards)
        self.sharding = sharding
        self.shape = tuple(int(s) for s in shape)
        live = [t for t in self.shards.values() if t is not None]
        self.dtype = dtype if dtype is not None else live[0].dtype
        want = sharding.shard_shape(self.shape)
        for d, t in self.shards.items():
            if t is not None and tuple(t.shape) != want:
                raise ValueError(f"shard on {d} has shape {tuple(t.shape)}, expected {want} for {sharding.spec}")

    @classmethod
    def _trusted(cls, shards: dict, sharding: NamedSharding, shape: tuple, dtype: torch.dtype) -> "DistArray":
        """Constructor for callers that have checked the shard shapes once already (the compiled step wraps the same
        outputs every step: thousands of arrays per step for a model with many parameters)."""
        self = object.__new__(cls)
        self.shards = shards
        self.sharding = sharding
        self.shape = shape
        self.dtype = dtype
        return self

    @property
    def mesh(self) -> Mesh:
        return self.sharding.mesh

    @property
    def spec(self) -> PartitionSpec:
        return self.sharding.spec

    @classmethod
    def from_global(cls, x: torch.Tensor, sharding: NamedSharding, devices: Iterable[Device] | None = None,
                    to_device: bool = True) -> "DistArray":
        """Shard a full tensor (every process passes the same ``x``)."""
        devices = list(devices) if devices is not None else list(sharding.mesh.flat_devices)
        shards = {}
        for d in devices:
            piece = x[sharding.device_index(d, x.shape)]
            piece = piece.to(d.torch_device) if to_device else piece
            shards[d] = piece.contiguous()
        return cls(shards, sharding, x.shape, x.dtype)

    def local(self, device: Device | None = None) -> torch.Tensor:
        if device is None:
            (device,) = [d for d, t in self.shards.items() if t is not None] if len(self.shards) == 1 else (None,)
            if device is None:
                raise ValueError("several shards are addressable; name the device")
        return self.shards[device]

    def to_global(self) -> torch.Tensor:
        """Assemble the full array (needs every distinct shard to be addressable)."""
        out = None
        covered = torch.zeros(self.shape, dtype=torch.bool) if self.shape else torch.zeros((), dtype=torch.bool)
        for d, t in self.shards.items():
            if t is None:
                continue
            if out is None:
                out = torch.empty(self.shape, dtype=self.dtype, device="cpu")
            idx = self.sharding.device_index(d, self.shape)
            out[idx] = t.detach().cpu()
            covered[idx] = True
        if out is None or not bool(covered.all()):
            raise ValueError("not every shard of the array is addressable from this process")
        return out

    def delete(self):
        for d in self.shards:
            self.shards[d] = None

    def is_deleted(self) -> bool:
        return all(t is None for t in self.shards.values())

    def __repr__(self):
        return f"DistArray(shape={self.shape}, dtype={self.dtype}, spec={self.spec}, mesh={self.mesh})"


# =============================================================================================
# MpmdSharding / MpmdArray
# =============================================================================================
@dataclasses.dataclass(frozen=True)
class MpmdSharding:
    mpmd_mesh: MpmdMesh
    mesh_ids: frozenset  # may be empty for unused arrays
    spec: PartitionSpec

    def __post_init__(self):
        object.__setattr__(self, "mesh_ids", frozenset(self.mesh_ids))
        # the stage sub-mesh has size 1 on the mpmd axis: it never shards anything
        object.__setattr__(self, "spec", filter_axes(PartitionSpec(*self.spec), {self.mpmd_mesh.mpmd_axis_name}))

    @property
    def sharding(self) -> NamedSharding:
        """Sharding over the union sub-mesh of all pipeline ranks in ``mesh_ids``."""
        ids = sorted(self.mesh_ids)
        return NamedSharding(self.mpmd_mesh.mpmd_submesh(ids).jax_mesh, self.spec)

    def local_sharding(self, mpmd_idx: int) -> NamedSharding:
        return NamedSharding(self.mpmd_mesh.unstack[mpmd_idx], self.spec)


class MpmdArray:
    """A logical array that exists on a *subset* of pipeline ranks (``mpmd_idxs``).

    Inside each of those ranks it is an SPMD :class:`DistArray` with ``spec``; when it lives on
    more than one rank the copies are replicas.  A process only holds data if it belongs to one of
    the ranks (``is_partially_addressable``); otherwise the object is metadata only.
    """

    def __init__(self, partially_addressable_arrays: Sequence[DistArray], mpmd_sharding: MpmdSharding,
                 shape: Sequence[int] | None = None, dtype: torch.dtype | None = None):
        mesh = mpmd_sharding.mpmd_mesh
        self._mpmd_sharding = mpmd_sharding
        self._mpmd_mesh = mesh
        self._mpmd_idxs = tuple(sorted(mpmd_sharding.mesh_ids))
        if mesh.jax_mesh.is_multi_process:
            assert len(partially_addressable_arrays) <= 1
        by_idx: dict[int, DistArray] = {}
        lookup = mesh.mpmd_idx_for_mesh
        for k, arr in enumerate(partially_addressable_arrays):
            idx = lookup.get(arr.mesh)
            if idx is None:
                raise ValueError(f"Argument array {k} {arr.shape} is not on a mesh that is part of mpmd_mesh={mesh.jax_mesh}")
            if idx not in mpmd_sharding.mesh_ids:
                raise ValueError(f"Argument array's ({k} {arr.shape}) mpmd_idx={idx} not in mpmd_idxs={self._mpmd_idxs}")
            if idx in by_idx:
                raise ValueError(f"Argument array {k} {arr.shape} already has a mpmd_idx={idx}")
            by_idx[idx] = arr
        self._arrays: "OrderedDict[int, DistArray]" = OrderedDict(sorted(by_idx.items()))
        if not self._arrays:
            assert shape is not None and dtype is not None
        else:
            first = next(iter(self._arrays.values()))
            shape = tuple(shape) if shape is not None else first.shape
            dtype = dtype if dtype is not None else first.dtype
            assert all(a.shape == tuple(shape) for a in self._arrays.values()), (shape, [a.shape for a in self._arrays.values()])
            assert all(a.dtype == dtype for a in self._arrays.values())
            low = mesh.lowering_mesh()
            want = rm_size1_axes(mpmd_sharding.spec, low)
            got = [rm_size1_axes(filter_axes(a.spec, {mesh.mpmd_axis_name}), low) for a in self._arrays.values()]
            assert all(g == want for g in got), (got, want)
        self._shape = tuple(int(s) for s in shape)
        self._dtype = dtype

    @classmethod
    def _trusted(cls, arrays: "OrderedDict[int, DistArray]", mpmd_sharding: MpmdSharding, idxs: tuple, shape: tuple,
                 dtype: torch.dtype) -> "MpmdArray":
        """Constructor without the consistency checks, for the compiled step's outputs (checked on its first call)."""
        self = object.__new__(cls)
        self._mpmd_sharding = mpmd_sharding
        self._mpmd_mesh = mpmd_sharding.mpmd_mesh
        self._mpmd_idxs = idxs
        self._arrays = arrays
        self._shape = shape
        self._dtype = dtype
        return self

    # -- metadata -------------------------------------------------------------------------------
    @property
    def spec(self) -> PartitionSpec:
        return self._mpmd_sharding.spec

    @property
    def shape(self) -> tuple[int, ...]:
        return self._shape

    @property
    def dtype(self) -> torch.dtype:
        return self._dtype

    @property
    def ndim(self) -> int:
        return len(self._shape)

    @property
    def mpmd_idxs(self) -> tuple[int, ...]:
        return self._mpmd_idxs

    @property
    def mpmd_sharding(self) -> MpmdSharding:
        return self._mpmd_sharding

    @property
    def sharding(self) -> NamedSharding:
        return self._mpmd_sharding.sharding

    @property
    def is_mpmd_replicated(self) -> bool:
        return len(self._mpmd_idxs) > 1

    @property
    def is_partially_addressable(self) -> bool:
        return len(self._arrays) > 0

    def __repr__(self):
        return f"MpmdArray(shape={self.shape}, dtype={self.dtype}, mpmd_idxs={self._mpmd_idxs}, spec={self.spec})"

    # -- data -----------------------------------------------------------------------------------
    def delete(self):
        assert self.is_partially_addressable, "Array is not partially addressable"
        assert not self.is_deleted(), "Array is deleted"
        for a in self._arrays.values():
            a.delete()

    def is_deleted(self) -> bool:
        assert self.is_partially_addressable, "Array is not partially addressable"
        flags = [a.is_deleted() for a in self._arrays.values()]
        assert any(flags) == all(flags)
        return flags[0]

    @property
    def to_mpmd_local_array(self):
        """The SPMD array of this process's pipeline rank (a list of them when one process drives
        several ranks), ``None`` if this process holds nothing."""
        if not self.is_partially_addressable:
            return None
        assert not self.is_deleted(), "Array is deleted"
        els = list(self._arrays.values())
        return els[0] if len(els) == 1 else els

    @property
    def first_mpmd_replica(self):
        """The local SPMD array iff it is the replica of the *lowest* owning rank — the one copy that a
        checkpoint writes."""
        if not self.is_partially_addressable:
            return None
        assert not self.is_deleted(), "Array is deleted"
        idx, arr = next(iter(self._arrays.items()))
        return arr if idx == self._mpmd_idxs[0] else None

    def local_tensor(self, mpmd_idx: int | None = None, device: Device | None = None) -> torch.Tensor | None:
        """The shard tensor on ``device`` (default: the only addressable one) of rank ``mpmd_idx``."""
        if not self.is_partially_addressable:
            return None
        arr = self._arrays[mpmd_idx] if mpmd_idx is not None else next(iter(self._arrays.values()))
        if device is None:
            live = [d for d, t in arr.shards.items() if t is not None]
            device = live[0]
        return arr.shards[device]

    def __int__(self):
        assert self.is_partially_addressable, "Array is not partially addressable"
        return int(self.local_tensor())

    def __float__(self):
        assert self.is_partially_addressable, "Array is not partially addressable"
        return float(self.local_tensor())

    def __format__(self, format_spec):
        assert self.is_partially_addressable, "Array is not partially addressable"
        t = self.local_tensor()
        return format(t.item() if t.numel() == 1 else t, format_spec)

    def block_until_ready(self):
        for a in self._arrays.values():
            for t in a.shards.values():
                if t is not None and t.is_cuda:
                    torch.cuda.current_stream(t.device).synchronize()
        return self


def _to_global_array(arr: MpmdArray) -> DistArray | None:
    """All addressable shards of ``arr`` as one DistArray over the union sub-mesh (reference:
    ``_to_global_jax_array``, array.py:265-293)."""
    if not arr.is_partially_addressable:
        return None
    shards = {}
    for a in arr._arrays.values():
        shards.update(a.shards)
    return DistArray(shards, arr.sharding, arr.shape, arr.dtype)


# =============================================================================================
# Resharding
# =============================================================================================
def _box_intersect(a: tuple[slice, ...], b: tuple[slice, ...]):
    out = []
    for sa, sb in zip(a, b):
        lo, hi = max(sa.start, sb.start), min(sa.stop, sb.stop)
        if lo >= hi:
            return None
        out.append(slice(lo, hi))
    return tuple(out)


def _rel(box, origin):
    return tuple(slice(b.start - o.start, b.stop - o.start) for b, o in zip(box, origin))


@dataclasses.dataclass
class CopyOp:
    src: Device
    dst: Device
    src_idx: tuple  # slices into the source shard
    dst_idx: tuple  # slices into the destination shard
    numel: int


def plan_reshard(shape: Sequence[int], src: NamedSharding, dst: NamedSharding) -> list[CopyOp]:
    """Box copies that build every ``dst`` shard out of ``src`` shards.  Among source replicas the one on
    the destination device itself is preferred, then the one on the same process, then the first."""
    shape = tuple(shape)
    src_boxes = [(d, src.device_index(d, shape)) for d in src.mesh.flat_devices]
    ops: list[CopyOp] = []
    for dd in dst.mesh.flat_devices:
        dbox = dst.device_index(dd, shape)
        # group source replicas by box
        by_box: dict[tuple, list[Device]] = {}
        for sd, sbox in src_boxes:
            by_box.setdefault(tuple((s.start, s.stop) for s in sbox), []).append(sd)
        for key, holders in by_box.items():
            sbox = tuple(slice(a, b) for a, b in key)
            inter = _box_intersect(sbox, dbox) if shape else ()
            if inter is None:
                continue
            holder = next((h for h in holders if h == dd), None) or next(
                (h for h in holders if h.process_index == dd.process_index), holders[0]
            )
            numel = 1
            for s in inter:
                numel *= s.stop - s.start
            ops.append(CopyOp(holder, dd, _rel(inter, sbox), _rel(inter, dbox), numel))
    return ops


def _my_process() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def reshard(arr: DistArray, dst: NamedSharding, donate: bool = False) -> DistArray:
    """Redistribute ``arr`` to ``dst`` (possibly a different mesh).  Collective over all processes that
    own a device of either mesh; every process must call it with the same arguments in the same order."""
    return reshard_group([arr], [dst], donate)[0]


def reshard_group(arrs: Sequence[DistArray], dsts: Sequence[NamedSharding], donate: bool = False) -> list[DistArray]:
    """Redistribute several arrays as one unit: the copies of all of them are posted together (one batch of
    point-to-point operations between processes), completed, and only then are the sources released.  What is in
    flight at once -- destination shards, staging buffers of strided pieces, and the sources -- is therefore bounded
    by the bytes of the group, which is how the memory-bounded groups of :func:`spmd_to_mpmd_reshard` bound peak
    memory.  Collective: same arguments, same order on every process."""
    import torch.distributed as dist

    me = _my_process()
    outs: list[dict] = []
    pending = []
    for arr, dst in zip(arrs, dsts):
        ops = plan_reshard(arr.shape, arr.sharding, dst)
        multi = arr.mesh.is_multi_process or dst.mesh.is_multi_process
        mine = lambda d, multi=multi: (not multi) or d.process_index == me
        out: dict[Device, torch.Tensor] = {}
        shard_shape = dst.shard_shape(arr.shape)
        for d in dst.mesh.flat_devices:
            if mine(d):
                out[d] = torch.empty(shard_shape, dtype=arr.dtype, device=d.torch_device)
        for op in ops:
            s_mine, d_mine = mine(op.src), mine(op.dst)
            if s_mine and d_mine:
                out[op.dst][op.dst_idx].copy_(arr.shards[op.src][op.src_idx])
            elif s_mine:
                buf = arr.shards[op.src][op.src_idx].contiguous()
                pending.append(dist.P2POp(dist.isend, buf, op.dst.process_index))
            elif d_mine:
                view = out[op.dst][op.dst_idx]
                buf = view if view.is_contiguous() else torch.empty(view.shape, dtype=arr.dtype, device=view.device)
                pending.append((dist.P2POp(dist.irecv, buf, op.src.process_index), view, buf))
        outs.append(out)
    if pending:
        p2p = [p if isinstance(p, dist.P2POp) else p[0] for p in pending]
        for w in dist.batch_isend_irecv(p2p):
            w.wait()
        for p in pending:
            if not isinstance(p, dist.P2POp) and p[1] is not p[2]:
                p[1].copy_(p[2])
    if donate:
        for arr in arrs:
            arr.delete()
    return [DistArray(out, dst, arr.shape, arr.dtype) for out, arr, dst in zip(outs, arrs, dsts)]


def _group_by_size_threshold(sizes: Sequence[int], order: Sequence[int], threshold: float) -> list[list[int]]:
    """Consecutive groups of ``order`` whose byte sums stay under ``threshold`` (a single array larger
    than the threshold forms its own group)."""
    groups, cur, tot = [], [], 0
    for i in order:
        if cur and tot + sizes[i] > threshold:
            groups.append(cur)
            cur, tot = [], 0
        cur.append(i)
        tot += sizes[i]
    if cur:
        groups.append(cur)
    return groups


def _interleaved_order(sizes: Sequence[int], targets: Sequence[int], n_ranks: int) -> list[int]:
    """Largest-first within each target rank, then round-robin over ranks, so that consecutive
    arrays land on different pipeline ranks and no rank's memory fills up first."""
    per_rank: dict[int, list[int]] = {r: [] for r in range(n_ranks)}
    for i, t in enumerate(targets):
        per_rank[t].append(i)
    for r in per_rank:
        per_rank[r].sort(key=lambda i: -sizes[i])
    order = []
    for tup in itertools.zip_longest(*[per_rank[r] for r in range(n_ranks)]):
        order.extend(i for i in tup if i is not None)
    return order


def _min_free_memory(devices: Iterable[Device]) -> float:
    free = float("inf")
    for d in devices:
        if d.kind == "cuda" and torch.cuda.is_available():
            free = min(free, torch.cuda.mem_get_info(d.torch_device)[0])
    if free == float("inf"):
        return free
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([free], dtype=torch.float64)
        if dist.get_backend() == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        free = float(t.item())
    return free


def logically_stacked(array: DistArray, comm_mesh: Mesh, mesh_axis_name: str, array_axis: int = 0,
                      strict: bool = False) -> DistArray:
    """View the per-rank copies of ``array`` as one array over ``comm_mesh`` with a new dimension at ``array_axis``
    that is split over ``mesh_axis_name`` (one entry per pipeline rank); no data moves: every addressable shard gains
    a dimension of size 1 (reference: array.py:553-600).

    With ``strict`` the spec must not mention ``mesh_axis_name`` already; otherwise that axis is dropped from it."""
    spec = array.sharding.spec
    mentioned = any(mesh_axis_name == e or (isinstance(e, tuple) and mesh_axis_name in e) for e in spec)
    if strict:
        assert not mentioned, f"axis_name {mesh_axis_name!r} already exists in spec {spec}"
    else:
        spec = filter_axes(spec, {mesh_axis_name})
    entries = list(spec) + [None] * (len(array.shape) - len(spec))
    new_spec = PartitionSpec(*entries[:array_axis], mesh_axis_name, *entries[array_axis:])
    n = comm_mesh.shape[mesh_axis_name]
    shape = (*array.shape[:array_axis], n, *array.shape[array_axis:])
    shards = {d: (None if t is None else t.unsqueeze(array_axis)) for d, t in array.shards.items()}
    return DistArray(shards, NamedSharding(comm_mesh, new_spec), shape, array.dtype)


def spmd_to_mpmd_reshard(mpmd_mesh: MpmdMesh, spmd_arrays: Any, mpmd_shardings: Any, threshold: float | None = None,
                         donate: bool = True) -> Any:
    """Move arrays sharded over the *whole* mesh (stage axis included) to the pipeline ranks that use
    them.

    ``spmd_arrays`` and ``mpmd_shardings`` are matching pytrees of :class:`DistArray` and
    :class:`MpmdSharding` (typically ``compiled.in_shardings``).  Arrays are processed in
    memory-bounded groups: largest first, interleaved over target ranks, each group at most
    ``threshold`` bytes (default: a third of the smallest free device memory).  A sharding with empty
    ``mesh_ids`` (an unused input) parks the array on rank 0.
    """
    from torch.utils import _pytree as pytree

    arrays, spec = pytree.tree_flatten(spmd_arrays, is_leaf=lambda x: isinstance(x, DistArray))
    shardings = pytree.tree_leaves(mpmd_shardings, is_leaf=lambda x: isinstance(x, MpmdSharding))
    if len(arrays) != len(shardings):
        raise ValueError(f"{len(arrays)} arrays but {len(shardings)} shardings")
    sizes = [int(torch.tensor(a.shape).prod().item()) * a.dtype.itemsize if a.shape else a.dtype.itemsize for a in arrays]
    targets = [min(s.mesh_ids) if s.mesh_ids else 0 for s in shardings]
    if threshold is None:
        threshold = _min_free_memory(mpmd_mesh.jax_mesh.flat_devices) / 3
    order = _interleaved_order(sizes, targets, mpmd_mesh.mpmd_dim)
    groups = _group_by_size_threshold(sizes, order, threshold)
    logger.info("spmd→mpmd reshard of %d arrays (%s) in %d groups", len(arrays), hbytes(sizes), len(groups))
    out: list[Any] = [None] * len(arrays)
    multi = mpmd_mesh.jax_mesh.is_multi_process
    me = _my_process()
    for group in groups:
        effs = []
        for i in group:
            sh = shardings[i]
            ids = sorted(sh.mesh_ids) if sh.mesh_ids else [0]
            effs.append((ids, MpmdSharding(mpmd_mesh, frozenset(ids), sh.spec)))
        # one group = one batch of copies: posted together, completed, sources released, then the next group
        moved_all = reshard_group([arrays[i] for i in group], [eff.sharding for _, eff in effs], donate=donate)
        for i, (ids, eff), moved in zip(group, effs, moved_all):
            locals_ = []
            for idx in ids:
                sub = mpmd_mesh.unstack[idx]
                shards = {d: moved.shards[d] for d in sub.flat_devices if d in moved.shards}
                if shards:
                    locals_.append(DistArray(shards, NamedSharding(sub, eff.spec), arrays[i].shape, arrays[i].dtype))
            out[i] = MpmdArray(locals_, eff, arrays[i].shape, arrays[i].dtype)
    return pytree.tree_unflatten(out, spec)


def mpmd_to_spmd_reshard(mpmd_mesh: MpmdMesh, mpmd_arrays: Any, spmd_shardings: Any) -> Any:
    """Inverse of :func:`spmd_to_mpmd_reshard`: every array becomes a :class:`DistArray` over the full
    mesh with the requested :class:`NamedSharding` (which may mention the stage axis).  The copy of
    the lowest owning rank is the source."""
    from torch.utils import _pytree as pytree

    arrays, spec = pytree.tree_flatten(mpmd_arrays, is_leaf=lambda x: isinstance(x, MpmdArray))
    shardings = pytree.tree_leaves(spmd_shardings, is_leaf=lambda x: isinstance(x, NamedSharding))
    if len(arrays) != len(shardings):
        raise ValueError(f"{len(arrays)} arrays but {len(shardings)} shardings")
    out = []
    for arr, sh in zip(arrays, shardings):
        first = arr.mpmd_idxs[0] if arr.mpmd_idxs else 0
        sub = mpmd_mesh.unstack[first]
        src_sh = NamedSharding(sub, arr.spec)
        shards = {}
        if arr.is_partially_addressable and first in arr._arrays:
            shards = dict(arr._arrays[first].shards)
        src = DistArray.__new__(DistArray)
        src.shards, src.sharding, src.shape, src.dtype = shards, src_sh, arr.shape, arr.dtype
        out.append(reshard(src, sh))
    return pytree.tree_unflatten(out, spec)
