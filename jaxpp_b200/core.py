"""``mpmd_jit_with_loop`` / ``mpmd_jit_by_yield``: capture, compile and run a pipelined step.

Public behaviour follows the reference's entry points (src/jaxpp/core.py:3854-3950): decorate the
train step, call it with (pytrees of) arrays, get back the same pytree structure with every leaf
an :class:`~jaxpp_b200.array.MpmdArray` that says on which pipeline ranks it lives; the compiled
object exposes ``in_shardings`` for placing inputs.  In one process the function drives every
rank itself (``GlobalMpmdFunction``, :3649-3793); in a one-process-per-device launch each process
runs only its rank's program (``ScalarMpmdFunction``, :3305-3447).
"""
from __future__ import annotations

import dataclasses
import os
from collections import OrderedDict
from typing import Any, Callable, Sequence

import torch
from torch.utils import _pytree as pytree

from .array import DistArray, MpmdArray, MpmdSharding
from .compiler.capture import ArgMeta, capture
from .compiler.lower import lower
from .compiler.program import Program
from .mesh import MpmdMesh, NamedSharding, PartitionSpec
from .runtime.executor import run_multi_controller, run_single_controller
from .schedules import BaseSchedule
from .utils import config, logger


@dataclasses.dataclass(frozen=True)
class ShapeDtypeStruct:
    """Stand-in for an array when only compiling (``.lower``): local shard shape and dtype."""

    shape: tuple
    dtype: torch.dtype


def _is_leaf(x) -> bool:
    return isinstance(x, (MpmdArray, ShapeDtypeStruct, DistArray))


def _leaf_meta(x, mesh: MpmdMesh) -> ArgMeta | None:
    if isinstance(x, torch.Tensor):
        return ArgMeta(tuple(x.shape), x.dtype)
    if isinstance(x, ShapeDtypeStruct):
        return ArgMeta(tuple(x.shape), x.dtype)
    if isinstance(x, MpmdArray):
        local = NamedSharding(mesh.lowering_mesh(), x.spec).shard_shape(x.shape)
        return ArgMeta(tuple(local), x.dtype)
    if isinstance(x, DistArray):
        return ArgMeta(tuple(x.sharding.shard_shape(x.shape)), x.dtype)
    return None


class CompiledMpmd:
    """A compiled step: the program plus what is needed to feed it and wrap its results."""

    def __init__(self, program: Program, mesh: MpmdMesh, in_spec, out_spec, tensor_positions, static_leaves, n_leaves,
                 in_specs_flat, out_specs_flat, donate_flat):
        self.program = program
        self.mesh = mesh
        self.in_spec, self.out_spec = in_spec, out_spec
        self.tensor_positions = tensor_positions
        self.static_leaves = static_leaves
        self.n_leaves = n_leaves
        self.in_specs_flat = in_specs_flat
        self.out_specs_flat = out_specs_flat
        self.donate_flat = donate_flat      # per tensor input: the caller gave the buffer up (donate_argnums/names)
        self._comm = None
        self.last_states = None

    # -- metadata -------------------------------------------------------------------------------
    @property
    def in_shardings(self):
        """Pytree (same structure as ``(args, kwargs)``) of :class:`MpmdSharding`: which pipeline
        ranks need each input.  Unused inputs have empty ``mesh_ids``."""
        leaves: list[Any] = [None] * self.n_leaves
        for k, pos in enumerate(self.tensor_positions):
            _, ranks = self.program.inputs[k]
            leaves[pos] = MpmdSharding(self.mesh, frozenset(ranks), self.in_specs_flat[k])
        for pos, v in self.static_leaves.items():
            leaves[pos] = None
        return pytree.tree_unflatten(leaves, self.in_spec)

    @property
    def out_shardings(self):
        leaves = []
        k = 0
        for o in self.program.outputs:
            if o[0] == "c":
                leaves.append(None)
            else:
                leaves.append(MpmdSharding(self.mesh, frozenset(o[2]), self.out_specs_flat[len(leaves)]))
        return pytree.tree_unflatten(leaves, self.out_spec)

    def dump(self, rank: int | None = None) -> str:
        return self.program.dump(rank)

    # -- execution --------------------------------------------------------------------------------
    def _devices(self):
        return [sub.flat_devices[0].torch_device for sub in self.mesh.unstack]

    def __call__(self, *args, record_events: bool = False, **kwargs):
        """Run the compiled step on the arguments it was compiled for (same pytree structure as at ``lower`` /
        ``compile`` time, as the reference's compiled functions are called, core.py:3649-3793).  The flat list of
        argument leaves is accepted as well."""
        if len(args) == 2 and isinstance(args[1], bool) and not kwargs:     # (leaves, record_events)
            args, record_events = args[:1], args[1]
        if len(args) == 1 and not kwargs and isinstance(args[0], list) and len(args[0]) == self.n_leaves:
            leaves = args[0]
        else:
            leaves, spec = pytree.tree_flatten((args, kwargs), is_leaf=_is_leaf)
            if spec != self.in_spec:
                raise TypeError("arguments do not have the structure this step was compiled for")
        with self.mesh:
            return self._run(leaves, record_events)

    def _run(self, leaves: list, record_events: bool = False):
        mesh = self.mesh
        prog = self.program
        tensors = [None if isinstance(leaves[p], ShapeDtypeStruct) else leaves[p] for p in self.tensor_positions]
        donated_arrays = [x for x, d in zip(tensors, self.donate_flat or ()) if d and isinstance(x, (MpmdArray, DistArray))]
        if not mesh.jax_mesh.is_multi_process and config.debug_force_mpmdify.value and mesh.unstack[0].size == 1:
            # one process, but the per-rank programs of the multi-process path: every pipeline rank runs its own
            # instruction list in a thread and talks to the others through in-process queues (reference:
            # JAXPP_DEBUG_FORCE_MPMDIFY, src/jaxpp/core.py:3817-3820)
            from .runtime.local_comm import run_scalarized_in_threads

            flat_in = []
            for x in tensors:
                if isinstance(x, MpmdArray):
                    x = x.local_tensor()
                elif isinstance(x, DistArray):
                    x = next(t for t in x.shards.values() if t is not None)
                flat_in.append(x)
            self._release_donated(donated_arrays)
            states, outs = run_scalarized_in_threads(prog, flat_in, self._devices(), record_events)
            self.last_states = states
            return self._wrap_outputs(outs)
        if not mesh.jax_mesh.is_multi_process:
            if mesh.unstack[0].size != 1:
                raise NotImplementedError(
                    "a single process can only drive stage sub-meshes of one device; launch one process per device"
                )
            devices = self._devices()
            flat_in = []
            for (vid, ranks), x in zip(prog.inputs, tensors):
                if isinstance(x, MpmdArray):
                    x = x.local_tensor()
                elif isinstance(x, DistArray):
                    x = next(t for t in x.shards.values() if t is not None)
                flat_in.append(x)
            self._release_donated(donated_arrays)
            states, outs = run_single_controller(prog, flat_in, devices, record_events)
            self.last_states = states
        else:
            from .runtime.comm import DistComm, ensure_groups

            rank = mesh.my_mpmd_axis_index
            device = mesh.my_device.torch_device
            if self._comm is None:
                self._comm = DistComm(mesh, device)
                ensure_groups(prog, self._comm)
            flat_in = []
            for x in tensors:
                if isinstance(x, MpmdArray):
                    x = x.local_tensor()
                elif isinstance(x, DistArray):
                    x = x.shards.get(mesh.my_device)
                flat_in.append(x)
            self._release_donated(donated_arrays)
            del tensors
            st, outs = run_multi_controller(prog, rank, flat_in, device, self._comm, record_events)
            self.last_states = [st]
        return self._wrap_outputs(outs)

    @staticmethod
    def _release_donated(arrays):
        """A donated argument is given up by the caller: the array objects passed in drop their buffers (they read as
        deleted afterwards, like a donated ``jax.Array``), so that the program's own deletes free the memory at the
        last use inside the step instead of when the caller lets go of the old state."""
        for a in arrays:
            try:
                if not a.is_deleted():
                    a.delete()
            except AssertionError:
                pass   # a metadata-only array of another pipeline rank: nothing to release here

    def _wrap_outputs(self, outs):
        """Flat program outputs -> the user's output tree of :class:`MpmdArray`.  What does not change from call to call
        (shardings, global shapes, the sub-mesh and device of every local piece) is worked out on the first call, which
        also builds the arrays through the checking constructors; later calls only attach the new tensors."""
        mesh = self.mesh
        plan = getattr(self, "_wrap_plan", None)
        wrapped = []
        if plan is None:
            plan = []
            low = mesh.lowering_mesh()
            for k, (o, val) in enumerate(zip(self.program.outputs, outs)):
                if o[0] == "c":
                    wrapped.append(val)
                    plan.append(None)
                    continue
                _, vid, ranks = o
                spec = self.out_specs_flat[k]
                info = self.program.values[vid]
                sharding = MpmdSharding(mesh, frozenset(ranks), spec)
                gshape = tuple(int(s * low.axis_size(sharding.spec.axes_of(d))) for d, s in enumerate(info.shape))
                pieces = {}
                for r in ranks:
                    sub = mesh.unstack[r]
                    dev = mesh.my_device if mesh.jax_mesh.is_multi_process else sub.flat_devices[0]
                    pieces[r] = (dev, NamedSharding(sub, sharding.spec))
                locals_ = [DistArray({pieces[r][0]: t}, pieces[r][1], gshape, info.dtype) for r, t in sorted(val.items())]
                wrapped.append(MpmdArray(locals_, sharding, gshape, info.dtype))   # checks shapes, dtypes and specs
                plan.append((sharding, tuple(sorted(sharding.mesh_ids)), gshape, info.dtype, pieces))
            self._wrap_plan = plan
            return pytree.tree_unflatten(wrapped, self.out_spec)
        for entry, val in zip(plan, outs):
            if entry is None:
                wrapped.append(val)
                continue
            sharding, idxs, gshape, dtype, pieces = entry
            arrays = OrderedDict()
            for r in sorted(val):
                dev, named = pieces[r]
                arrays[r] = DistArray._trusted({dev: val[r]}, named, gshape, dtype)
            wrapped.append(MpmdArray._trusted(arrays, sharding, idxs, gshape, dtype))
        return pytree.tree_unflatten(wrapped, self.out_spec)


class MpmdFunction:
    """The callable returned by :func:`mpmd_jit_with_loop` / :func:`mpmd_jit_by_yield`."""

    def __init__(self, fun: Callable, mpmd_mesh: MpmdMesh, with_loop: bool, in_specs=None, out_specs=None,
                 static_argnums: Sequence[int] = (), static_argnames: Sequence[str] = (),
                 donate_argnums: Sequence[int] = (), donate_argnames: Sequence[str] = (),
                 schedule: BaseSchedule | None = None, name: str | None = None, compiler_options=None):
        self.fun = fun
        self.mpmd_mesh = mpmd_mesh
        self.with_loop = with_loop
        self.in_specs = in_specs
        self.out_specs = out_specs
        self.static_argnums = tuple(static_argnums)
        self.static_argnames = tuple(static_argnames)
        self.donate_argnums = tuple(donate_argnums)
        self.donate_argnames = tuple(donate_argnames)
        self.schedule = schedule
        self.name = name or getattr(fun, "__name__", "step")
        self.compiler_options = dict(compiler_options or {})
        if self.compiler_options:
            # the reference forwards these to XLA; tasks here are kernel launches from generated Python, there is no
            # compiler to configure
            logger.warning("compiler_options %s have no effect: tasks are not XLA executables", sorted(self.compiler_options))
        self._cache: dict[Any, CompiledMpmd] = {}

    # -- compile -------------------------------------------------------------------------------
    def _prepare(self, args, kwargs):
        leaves, in_spec = pytree.tree_flatten((args, kwargs), is_leaf=_is_leaf)
        metas, static = [], {}
        for pos, leaf in enumerate(leaves):
            m = _leaf_meta(leaf, self.mpmd_mesh)
            if m is None:
                static[pos] = leaf
            else:
                metas.append(m)
        # Every leaf that is not an array is static: it is baked into the program and is part of the cache key (a new
        # value compiles a new program).  static_argnums / static_argnames are therefore only checked: an argument
        # named static must not contain arrays (the reference requires static arguments to be hashable constants).
        key = (in_spec, tuple(metas), tuple(sorted((p, repr(v)) for p, v in static.items())))
        return leaves, in_spec, metas, static, key

    def _arg_leaf_ranges(self, args, kwargs) -> tuple[dict, dict]:
        """Flat leaf positions of every positional and keyword argument in the flattening of ``(args, kwargs)``."""
        pos, by_num, by_name = 0, {}, {}
        for i, a in enumerate(args):
            n = len(pytree.tree_leaves(a, is_leaf=_is_leaf))
            by_num[i] = range(pos, pos + n)
            pos += n
        for k, v in kwargs.items():
            n = len(pytree.tree_leaves(v, is_leaf=_is_leaf))
            by_name[k] = range(pos, pos + n)
            pos += n
        return by_num, by_name

    def _selected_leaves(self, args, kwargs, nums, names, what: str) -> set:
        by_num, by_name = self._arg_leaf_ranges(args, kwargs)
        out: set = set()
        for i in nums:
            if i not in by_num:
                raise ValueError(f"{what}_argnums names positional argument {i} but the call has {len(args)}")
            out.update(by_num[i])
        for k in names:
            if k in by_name:
                out.update(by_name[k])
        return out

    def lower(self, *args, **kwargs) -> CompiledMpmd:
        leaves, in_spec, metas, static, key = self._prepare(args, kwargs)
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        mesh = self.mpmd_mesh
        config.warn_about_flags_without_effect(logger)
        tensor_positions = [p for p in range(len(leaves)) if p not in static]
        static_named = self._selected_leaves(args, kwargs, self.static_argnums, self.static_argnames, "static")
        bad = sorted(p for p in static_named if p not in static)
        if bad:
            raise TypeError(f"static_argnums / static_argnames name an argument that contains arrays (flat leaves {bad}); "
                            "static arguments must be Python constants")
        donated_leaves = self._selected_leaves(args, kwargs, self.donate_argnums, self.donate_argnames, "donate")
        donate_flat = [p in donated_leaves for p in tensor_positions]
        with mesh:
            cap = capture(self.fun, in_spec, metas, static, len(leaves))
            if self.with_loop and cap.trace.n_loops != 1:
                raise AssertionError("mpmd_jit_with_loop needs exactly one treduce loop in the function")
            program = lower(cap, mesh.mpmd_dim, self.schedule, self.name,
                            donated_inputs={k for k, d in enumerate(donate_flat) if d})
        in_specs_flat = self._flat_specs(self.in_specs, (args, kwargs), len(metas), leaves, tensor_positions)
        out_leaves_n = len(program.outputs)
        out_specs_flat = self._flat_out_specs(self.out_specs, cap.out_spec, out_leaves_n)
        compiled = CompiledMpmd(program, mesh, in_spec, cap.out_spec, tensor_positions, static, len(leaves),
                                in_specs_flat, out_specs_flat, donate_flat)
        self._cache[key] = compiled
        if config.dump_dir.value:
            self._dump(compiled)
        logger.info("compiled %s: %s", self.name, program.stats())
        return compiled

    compile = lower   # name under which the reference's jitted functions expose it (core.py:3471)

    def _flat_specs(self, specs, tree, n, leaves, tensor_positions):
        out = []
        if specs is not None:
            flat = pytree.tree_leaves(specs, is_leaf=lambda x: isinstance(x, PartitionSpec) or x is None)
            flat = [s if s is not None else PartitionSpec() for s in flat]
            if len(flat) == n:
                return flat
            raise ValueError(f"in_specs has {len(flat)} leaves but the function takes {n} array arguments")
        for p in tensor_positions:
            leaf = leaves[p]
            out.append(leaf.spec if isinstance(leaf, (MpmdArray, DistArray)) else PartitionSpec())
        return out

    def _flat_out_specs(self, specs, out_spec, n):
        if specs is None:
            return [PartitionSpec()] * n
        flat = pytree.tree_leaves(specs, is_leaf=lambda x: isinstance(x, PartitionSpec) or x is None)
        flat = [s if s is not None else PartitionSpec() for s in flat]
        if len(flat) != n:
            raise ValueError(f"out_specs has {len(flat)} leaves but the function returns {n}")
        return flat

    def _dump(self, compiled: CompiledMpmd):
        d = config.dump_dir.value
        os.makedirs(d, exist_ok=True)
        proc = int(os.environ.get("RANK", "0"))
        with open(os.path.join(d, f"{self.name}.global.{proc}.program.txt"), "w") as f:
            f.write(compiled.dump())
        for r in range(compiled.program.n_ranks):
            with open(os.path.join(d, f"{self.name}.local.{proc}.rank{r}.program.txt"), "w") as f:
                f.write(compiled.dump(r))

    # -- run -------------------------------------------------------------------------------------
    def __call__(self, *args, **kwargs):
        leaves, in_spec, metas, static, key = self._prepare(args, kwargs)
        compiled = self._cache.get(key)
        if compiled is None:
            compiled = self.lower(*args, **kwargs)
        return compiled(leaves)


def _check_specs(in_specs, in_shardings, out_specs, out_shardings):
    if in_specs is not None and in_shardings is not None:
        raise ValueError("Only one of `in_specs` and `in_shardings` can be given")
    if out_specs is not None and out_shardings is not None:
        raise ValueError("Only one of `out_specs` and `out_shardings` can be given")


def _specs_of(shardings):
    if shardings is None:
        return None
    return pytree.tree_map(lambda s: s.spec if s is not None else None, shardings,
                           is_leaf=lambda x: isinstance(x, (MpmdSharding, NamedSharding)) or x is None)


def mpmd_jit_with_loop(fun: Callable, mpmd_mesh: MpmdMesh, *, in_shardings=None, in_specs=None, out_shardings=None,
                       out_specs=None, static_argnums=(), static_argnames=(), donate_argnums=(), donate_argnames=(),
                       compiler_options=None, name: str | None = None) -> MpmdFunction:
    """Compile a train step that contains exactly one :func:`~jaxpp_b200.training.treduce` loop into
    one program per pipeline rank of ``mpmd_mesh`` (reference: core.py:3892-3923).

    ``donate_argnums`` / ``donate_argnames``: the caller gives these arguments' buffers up.  The program frees each of
    them after its last use on every rank (instead of keeping program inputs alive for the whole step), and array
    objects passed for them read as deleted after the call (reference: core.py:1732-1809, 3892-3923).
    ``static_argnums`` / ``static_argnames``: every non-array leaf is a compile-time constant here anyway; the named
    arguments are checked to contain no arrays.  ``compiler_options`` are kept on the returned object and otherwise
    unused (there is no XLA executable to configure)."""
    _check_specs(in_specs, in_shardings, out_specs, out_shardings)
    return MpmdFunction(fun, mpmd_mesh, True, in_specs if in_specs is not None else _specs_of(in_shardings),
                        out_specs if out_specs is not None else _specs_of(out_shardings), static_argnums,
                        static_argnames, donate_argnums, donate_argnames, name=name, compiler_options=compiler_options)


def mpmd_jit_by_yield(fun: Callable, mpmd_mesh: MpmdMesh, *, in_shardings=None, in_specs=None, out_shardings=None,
                      out_specs=None, static_argnums=(), static_argnames=(), donate_argnums=(), donate_argnames=(),
                      compiler_options=None, name: str | None = None) -> MpmdFunction:
    """Compile a function without a microbatch loop: stage ``s`` (delimited by ``mark_stage_end``) runs
    on pipeline rank ``s % mpmd_dim`` (reference: core.py:3926-3950)."""
    _check_specs(in_specs, in_shardings, out_specs, out_shardings)
    return MpmdFunction(fun, mpmd_mesh, False, in_specs if in_specs is not None else _specs_of(in_shardings),
                        out_specs if out_specs is not None else _specs_of(out_shardings), static_argnums,
                        static_argnames, donate_argnums, donate_argnames, name=name, compiler_options=compiler_options)


# ---------------------------------------------------------------------------------------------------
def value_and_grad(fun: Callable, argnums: int | Sequence[int] = 0, has_aux: bool = False,
                   grad_dtype: torch.dtype | None = None) -> Callable:
    """``jax.value_and_grad`` for pytrees of tensors, built on ``torch.autograd.grad`` so that it can
    be captured: the differentiated arguments are detached copies that require grad.

    ``grad_dtype``: dtype the gradients are delivered in (default: each argument's own dtype).  With
    ``torch.float32`` a weight gradient that a GEMM epilogue wrote in fp32 reaches the caller, and the
    accumulation over microbatches, without a round trip through the parameter's bf16."""
    nums = (argnums,) if isinstance(argnums, int) else tuple(argnums)

    def wrapped(*args, **kwargs):
        args = list(args)
        flat_all, specs = [], []
        for n in nums:
            leaves, spec = pytree.tree_flatten(args[n])
            leaves = [l.detach().requires_grad_(True) if l.is_floating_point() else l for l in leaves]
            if grad_dtype is not None:
                for l in leaves:
                    if l.requires_grad:
                        l.grad_dtype = grad_dtype
            args[n] = pytree.tree_unflatten(leaves, spec)
            flat_all.append(leaves)
            specs.append(spec)
        with torch.enable_grad():
            out = fun(*args, **kwargs)
            value, aux = out if has_aux else (out, None)
            diff = [l for leaves in flat_all for l in leaves if l.requires_grad]
            grads = torch.autograd.grad(value, diff, allow_unused=True)
        it = iter(grads)
        trees = []
        for leaves, spec in zip(flat_all, specs):
            gl = []
            for l in leaves:
                if l.requires_grad:
                    g = next(it)
                    gl.append(g if g is not None else torch.zeros_like(l, dtype=grad_dtype or l.dtype))
                else:
                    gl.append(None)
            trees.append(pytree.tree_unflatten(gl, spec))
        g_out = trees[0] if isinstance(argnums, int) else tuple(trees)
        value = value.detach()
        return ((value, aux), g_out) if has_aux else (value, g_out)

    return wrapped
