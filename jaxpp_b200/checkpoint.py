"""Checkpoint / resume with a layout-independent on-disk format.

The reference has no checkpointing; its intended path is ``mpmd_to_spmd_reshard`` → an SPMD checkpointer →
``spmd_to_mpmd_reshard`` (examples/mpmd_reshard.py:89-111).  Here the format is defined directly:

    <dir>/step_<n>/manifest.json            pytree path → {shape, dtype, spec, mesh_ids, shards:[{file, index}]}
    <dir>/step_<n>/<path>.<k>.bin           raw little-endian bytes of one shard (C order)
    <dir>/step_<n>/extra.json               step counter, config, data cursor, RNG seeds … (user dict)

Only the first replica of every shard is written (lowest owning pipeline rank, and inside it the device whose
coordinates on all non-sharding mesh axes are 0).  Writers create the step directory under a temporary name;
after a barrier rank 0 merges the per-process manifests, fsyncs and renames — readers never see a partial
checkpoint.  Loading assembles, for every device, the hyper-rectangle it needs from whichever shard files
intersect it, so a checkpoint written with one PP x TP x DP layout restores into another.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Any, Mapping

import numpy as np
import torch
from torch.utils import _pytree as pytree

from .array import DistArray, MpmdArray, MpmdSharding, _box_intersect, _rel
from .mesh import Device, MpmdMesh, NamedSharding, PartitionSpec

_DTYPES = {
    "float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "int64": torch.int64,
    "int32": torch.int32, "uint8": torch.uint8, "float64": torch.float64, "bool": torch.bool,
}
_VIEW = {torch.bfloat16: torch.int16, torch.bool: torch.uint8}  # numpy has no bf16: reinterpret


def _dist():
    import torch.distributed as dist

    return dist if dist.is_available() and dist.is_initialized() else None


def _rank() -> int:
    d = _dist()
    return d.get_rank() if d else 0


def _barrier():
    d = _dist()
    if d:
        d.barrier()


def _paths(tree) -> list[str]:
    flat, _ = pytree.tree_flatten_with_path(tree, is_leaf=lambda x: isinstance(x, (MpmdArray, DistArray)))
    out = []
    for path, _leaf in flat:
        parts = []
        for k in path:
            parts.append(str(getattr(k, "key", getattr(k, "idx", getattr(k, "name", k)))))
        out.append("/".join(parts))
    return out


def _to_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.dtype in _VIEW:
        t = t.view(_VIEW[t.dtype])
    return t.numpy().tobytes()


def _spec_json(spec: PartitionSpec):
    return [list(p) if isinstance(p, tuple) else p for p in spec]


def _spec_from_json(js) -> PartitionSpec:
    return PartitionSpec(*[tuple(p) if isinstance(p, list) else p for p in js])


def _is_first_replica(device: Device, sharding: NamedSharding) -> bool:
    used = set(sharding.spec.all_axes())
    coord = dict(zip(sharding.mesh.axis_names, sharding.mesh.device_coords[device]))
    return all(c == 0 for a, c in coord.items() if a not in used)


def save(directory: str, step: int, tree: Any, mesh: MpmdMesh, extra: Mapping | None = None) -> str:
    """Write ``tree`` (leaves: :class:`MpmdArray`, or plain tensors = replicated on every rank) for ``step``.
    Collective over all processes; returns the final directory."""
    final = os.path.join(directory, f"step_{step:08d}")
    tmp = final + ".tmp"
    me = _rank()
    if me == 0:
        if os.path.exists(tmp):
            shutil.rmtree(tmp)
        os.makedirs(tmp)
    _barrier()
    leaves = pytree.tree_leaves(tree, is_leaf=lambda x: isinstance(x, (MpmdArray, DistArray)))
    names = _paths(tree)
    entries: dict[str, dict] = {}
    for name, leaf in zip(names, leaves):
        fname = name.replace("/", ".")
        if isinstance(leaf, torch.Tensor):  # replicated everywhere: process 0 writes it whole
            entry = {"shape": list(leaf.shape), "dtype": str(leaf.dtype).replace("torch.", ""), "spec": [],
                     "mesh_ids": list(range(mesh.mpmd_dim)), "shards": []}
            if me == 0:
                f = f"{fname}.0.bin"
                with open(os.path.join(tmp, f), "wb") as fh:
                    fh.write(_to_bytes(leaf))
                entry["shards"].append({"file": f, "index": [[0, s] for s in leaf.shape]})
            entries[name] = entry
            continue
        assert isinstance(leaf, MpmdArray), f"{name}: cannot checkpoint {type(leaf)}"
        entry = {"shape": list(leaf.shape), "dtype": str(leaf.dtype).replace("torch.", ""), "spec": _spec_json(leaf.spec),
                 "mesh_ids": list(leaf.mpmd_idxs), "shards": []}
        first = leaf.first_mpmd_replica
        if first is not None:
            for dev, t in first.shards.items():
                if t is None or not _is_first_replica(dev, first.sharding):
                    continue
                idx = first.sharding.device_index(dev, leaf.shape)
                f = f"{fname}.{dev.id}.bin"
                with open(os.path.join(tmp, f), "wb") as fh:
                    fh.write(_to_bytes(t))
                entry["shards"].append({"file": f, "index": [[s.start, s.stop] for s in idx]})
        entries[name] = entry
    with open(os.path.join(tmp, f"manifest.rank{me}.json"), "w") as fh:
        json.dump(entries, fh)
        fh.flush()
        os.fsync(fh.fileno())
    _barrier()
    if me == 0:
        merged: dict[str, dict] = {}
        for f in sorted(os.listdir(tmp)):
            if not f.startswith("manifest.rank"):
                continue
            part = json.load(open(os.path.join(tmp, f)))
            for name, e in part.items():
                if name not in merged:
                    merged[name] = e
                else:
                    merged[name]["shards"].extend(e["shards"])
            os.remove(os.path.join(tmp, f))
        for name, e in merged.items():
            covered = sum(int(np.prod([b - a for a, b in s["index"]])) if s["index"] else 1 for s in e["shards"])
            total = int(np.prod(e["shape"])) if e["shape"] else 1
            if covered != total:
                raise RuntimeError(f"checkpoint entry {name}: shards cover {covered} of {total} elements")
        with open(os.path.join(tmp, "manifest.json"), "w") as fh:
            json.dump({"step": step, "entries": merged}, fh, indent=1)
            fh.flush()
            os.fsync(fh.fileno())
        with open(os.path.join(tmp, "extra.json"), "w") as fh:
            json.dump(dict(extra or {}), fh)
            fh.flush()
            os.fsync(fh.fileno())
        if os.path.exists(final):
            shutil.rmtree(final)
        os.rename(tmp, final)
        dfd = os.open(directory, os.O_RDONLY)
        try:
            os.fsync(dfd)
        finally:
            os.close(dfd)
    _barrier()
    return final


def latest_step(directory: str) -> int | None:
    if not os.path.isdir(directory):
        return None
    steps = [int(d[5:]) for d in os.listdir(directory) if d.startswith("step_") and not d.endswith(".tmp")
             and os.path.exists(os.path.join(directory, d, "manifest.json"))]
    return max(steps) if steps else None


def _read_box(ckpt_dir: str, entry: dict, box: tuple[slice, ...], dtype: torch.dtype) -> torch.Tensor:
    shape = tuple(s.stop - s.start for s in box)
    out = torch.empty(shape, dtype=dtype)
    filled = 0
    store = _VIEW.get(dtype, dtype)
    np_dtype = torch.empty(0, dtype=store).numpy().dtype
    for sh in entry["shards"]:
        sbox = tuple(slice(a, b) for a, b in sh["index"])
        inter = _box_intersect(sbox, box) if shape else ()
        if inter is None:
            continue
        sshape = tuple(b - a for a, b in sh["index"])
        arr = np.memmap(os.path.join(ckpt_dir, sh["file"]), dtype=np_dtype, mode="r", shape=sshape)
        piece = torch.from_numpy(np.array(arr[_rel(inter, sbox)] if shape else arr))
        if store is not dtype:
            piece = piece.view(dtype)
        if shape:
            out[_rel(inter, box)] = piece
            filled += piece.numel()
        else:
            out.copy_(piece.reshape(()))
            filled += 1
    want = out.numel()
    if filled != want:
        raise RuntimeError(f"checkpoint shards cover {filled} of {want} elements of the requested block")
    return out


def load(directory: str, step: int | None, target: Any, mesh: MpmdMesh) -> tuple[Any, dict]:
    """Restore into the layout described by ``target``: a pytree with the saved structure whose leaves are
    :class:`MpmdSharding` (→ :class:`MpmdArray`), or ``None`` (→ full tensor on every process).
    Returns ``(tree, extra)``."""
    if step is None:
        step = latest_step(directory)
        if step is None:
            raise FileNotFoundError(f"no complete checkpoint under {directory}")
    ckpt = os.path.join(directory, f"step_{step:08d}")
    manifest = json.load(open(os.path.join(ckpt, "manifest.json")))["entries"]
    extra = json.load(open(os.path.join(ckpt, "extra.json")))
    is_leaf = lambda x: isinstance(x, MpmdSharding) or x is None
    leaves, spec = pytree.tree_flatten(target, is_leaf=is_leaf)
    flat, _ = pytree.tree_flatten_with_path(target, is_leaf=is_leaf)
    names = []
    for path, _ in flat:
        names.append("/".join(str(getattr(k, "key", getattr(k, "idx", getattr(k, "name", k)))) for k in path))
    local = set(mesh.local_devices)
    out = []
    for name, tgt in zip(names, leaves):
        if name not in manifest:
            raise KeyError(f"checkpoint has no entry {name!r}")
        e = manifest[name]
        dtype = _DTYPES[e["dtype"]]
        shape = tuple(e["shape"])
        if tgt is None:
            out.append(_read_box(ckpt, e, tuple(slice(0, s) for s in shape), dtype))
            continue
        arrays = []
        for idx in sorted(tgt.mesh_ids):
            sub = mesh.unstack[idx]
            sh = NamedSharding(sub, tgt.spec)
            shards = {}
            for dev in sub.flat_devices:
                if dev in local:
                    shards[dev] = _read_box(ckpt, e, sh.device_index(dev, shape), dtype).to(dev.torch_device)
            if shards:
                arrays.append(DistArray(shards, sh, shape, dtype))
        out.append(MpmdArray(arrays, tgt, shape, dtype))
    return pytree.tree_unflatten(out, spec), extra
