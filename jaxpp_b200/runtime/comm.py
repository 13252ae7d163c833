"""Inter-rank communication for the multi-controller executor.

``DistComm`` moves activations and gradients between pipeline ranks with point-to-point messages
through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo on CPU ranks) and runs cross-stage
collectives on sub-groups.  It keeps the semantics of the reference's p2p backend
(src/jaxpp/dime2.py:258-345): all arrays of one transfer go out as one batch, communication runs on
side streams, a receive only blocks the compute stream when a task actually consumes the buffer,
and a sent buffer is kept alive until its ``send_done``.  Peers are positional: device ``k`` of one
stage sub-mesh talks to device ``k`` of the other, so both sides must shard identically (:149-152).
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.distributed as dist

from ..compiler.program import AllGather, Program, SendDone, Transfer
from .. import fault
from ..mesh import MpmdMesh


class DistComm:
    def __init__(self, mesh: MpmdMesh, device: torch.device):
        self.mesh = mesh
        self.device = device
        self.rank = mesh.my_mpmd_axis_index
        me = mesh.my_device
        sub = mesh.unstack[self.rank]
        self.pos_in_stage = list(sub.flat_devices).index(me)
        self.cuda = device.type == "cuda"
        self.pending_recv: dict[int, tuple] = {}  # vid → (work list, event)
        self.inflight_send: dict[int, tuple] = {}  # tid → (tensors, works)
        self.groups: dict[tuple, object] = {}
        self.p2p_groups: dict[tuple, object] = {}  # (src pipeline rank, dst pipeline rank) → 2-process group
        self.native_p2p = None                     # NcclP2P when JAXPP_B200_P2P=native
        if dist.is_available() and dist.is_initialized():
            mesh.create_process_groups()  # no-op when the mesh was made by MpmdMesh.create
        if self.cuda:
            self.send_stream = torch.cuda.Stream(device)
            self.recv_stream = torch.cuda.Stream(device)

    def _tag(self, tid: int, k: int) -> int:
        """Message tag: gloo needs a distinct tag per message in flight between a pair; NCCL ignores tags."""
        return 0 if self.cuda else (tid * 64 + k) % (1 << 30)

    def peer(self, mpmd_rank: int) -> int:
        """Global process rank of my positional counterpart in pipeline rank ``mpmd_rank``."""
        return self.mesh.unstack[mpmd_rank].flat_devices[self.pos_in_stage].process_index

    # -- step bracket -----------------------------------------------------------------------------
    def begin_step(self, st):
        self.pending_recv.clear()

    def end_step(self, st):
        for tid in list(self.inflight_send):
            self._finish_send(tid)
        self.before_use(st, list(self.pending_recv))


    # -- p2p ------------------------------------------------------------------------------------------
    def send(self, st, ins: Transfer, prog: Program):
        if fault._PLAN[0] is not None and fault.transfer_action(self.rank, ins.tid) == "drop":
            return  # injected fault: the message is never sent
        peer = self.peer(ins.dst)
        tensors = [st.env[v].contiguous() for v in ins.vids]
        if self.cuda and self.native_p2p is not None:
            ready = torch.cuda.Event()
            ready.record()
            works = [self.native_p2p.send(peer, tensors, ready)]  # an event: the transfer's completion
        elif self.cuda:
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(self.send_stream):
                self.send_stream.wait_event(ready)
                g = self.p2p_groups.get((self.rank, ins.dst))
                works = dist.batch_isend_irecv([dist.P2POp(dist.isend, t, peer, group=g) for t in tensors])
        else:
            # gloo: one message per transfer (all arrays packed into one byte buffer)
            packed = torch.cat([t.reshape(-1).view(torch.uint8) for t in tensors]) if len(tensors) > 1 else tensors[0]
            tensors = [packed]
            works = [dist.isend(packed, peer, tag=self._tag(ins.tid, 0))]
        self.inflight_send[ins.tid] = (tensors, works)

    def recv(self, st, ins: Transfer, prog: Program):
        peer = self.peer(ins.rank)
        bufs = []
        for v in ins.vids:
            info = prog.values[v]
            bufs.append(torch.empty(info.shape, dtype=info.dtype, device=self.device))
        if self.cuda and self.native_p2p is not None:
            ready = torch.cuda.Event()
            ready.record()  # the buffers' allocation point on the compute stream
            done = self.native_p2p.recv(peer, bufs, ready)
            token = [[], done, False]
        elif self.cuda:
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(self.recv_stream):
                self.recv_stream.wait_event(ready)
                g = self.p2p_groups.get((ins.rank, self.rank))
                works = dist.batch_isend_irecv([dist.P2POp(dist.irecv, b, peer, group=g) for b in bufs])
                for w in works:
                    w.wait()  # orders recv_stream after the NCCL stream; does not block the host
                done = torch.cuda.Event()
                done.record()
            token = [works, done, False]
        else:
            if len(bufs) > 1:
                sizes = [b.numel() * b.element_size() for b in bufs]
                packed = torch.empty(sum(sizes), dtype=torch.uint8)
                views, off = [], 0
                for b, n in zip(bufs, sizes):
                    views.append(packed[off:off + n].view(b.dtype).view(b.shape))
                    off += n
                bufs = views
                works = [dist.irecv(packed, peer, tag=self._tag(ins.tid, 0))]
            else:
                works = [dist.irecv(bufs[0], peer, tag=self._tag(ins.tid, 0))]
            token = [works, None, False]
        for v, b in zip(ins.vids, bufs):
            st.env[v] = b
            self.pending_recv[v] = token

    def before_use(self, st, vids: Iterable[int]):
        """Make the consumer wait for any pending receive among ``vids``."""
        for v in vids:
            token = self.pending_recv.pop(v, None)
            if token is None:
                continue
            works, done, waited = token
            if waited:  # another array of the same transfer already waited (a gloo work must be waited once)
                continue
            token[2] = True
            if done is not None:
                torch.cuda.current_stream(self.device).wait_event(done)
            else:
                for w in works:
                    w.wait()

    def send_done(self, st, ins: SendDone):
        self._finish_send(ins.tid)

    def _finish_send(self, tid: int):
        item = self.inflight_send.pop(tid, None)
        if item is None:
            return
        tensors, works = item
        if self.cuda and self.native_p2p is not None:
            return  # the payloads were recorded on the pair's stream when the send was enqueued
        if self.cuda:
            with torch.cuda.stream(self.send_stream):
                for w in works:
                    w.wait()
            for t in tensors:
                t.record_stream(self.send_stream)
        else:
            for w in works:
                w.wait()

    # -- cross-stage collectives --------------------------------------------------------------------------
    def _group(self, ranks):
        """Process group of my positional counterparts in pipeline ranks ``ranks``.  Groups for all
        positions are created together (``new_group`` is collective over the whole world)."""
        key = tuple(ranks)
        if key not in self.groups:
            mine = None
            n_pos = self.mesh.unstack[0].size
            for pos in range(n_pos):
                procs = [self.mesh.unstack[r].flat_devices[pos].process_index for r in ranks]
                g = dist.new_group(ranks=procs)
                if pos == self.pos_in_stage:
                    mine = g
            self.groups[key] = mine
        return self.groups[key]

    def all_reduce(self, buf: torch.Tensor, ranks):
        """Sum over my positional counterparts in pipeline ranks ``ranks``.  Large CUDA tensors (tied-weight
        gradients) go through the one-kernel all-reduce over NVLink peer memory, the rest through NCCL / gloo."""
        group = self._group(ranks)
        if self.cuda and buf.dtype in (torch.float32, torch.bfloat16):
            from ..parallel import fused
            from ..utils import config

            if (buf.numel() * buf.element_size() >= fused.AR_MIN_BYTES and config.use_fused_collectives.value
                    and config.use_native_kernels.value):
                procs = [self.mesh.unstack[r].flat_devices[self.pos_in_stage].process_index for r in ranks]
                return fused.all_reduce_group(buf, group, procs)
        dist.all_reduce(buf, group=group)
        return buf

    def all_gather(self, st, ins: AllGather, prog: Program):
        """Concatenate operands that live on different pipeline ranks (``cross_mpmd_stack``): ONE all-gather over
        the group.  Every rank packs the operands it owns into a flat buffer; operand shapes are static (all equal
        along every dimension, the output's extent along ``axis`` divided by the operand count), so every rank knows
        every pack's size, and packs are padded to the largest one."""
        group = self._group(ins.ranks)
        info = prog.values[ins.out]
        n = len(ins.owners)
        shape = list(info.shape)
        shape[ins.axis] = info.shape[ins.axis] // n
        numel = 1
        for s_ in shape:
            numel *= s_
        owned = {r: [p for p, o in enumerate(ins.owners) if o == r] for r in ins.ranks}
        width = max(len(ps) for ps in owned.values()) * numel
        pack = torch.zeros(width, dtype=info.dtype, device=self.device)
        for k, p in enumerate(owned[self.rank]):
            pack[k * numel:(k + 1) * numel].copy_(st.env[ins.local[p]].reshape(-1))
        every = torch.empty(len(ins.ranks) * width, dtype=info.dtype, device=self.device)
        dist.all_gather_into_tensor(every, pack, group=group)
        parts: list = [None] * n
        for g, r in enumerate(ins.ranks):
            for k, p in enumerate(owned[r]):
                parts[p] = every[g * width + k * numel:g * width + (k + 1) * numel].view(shape)
        return torch.cat(parts, dim=ins.axis)


_P2P_GROUPS: dict[tuple, object] = {}
_NATIVE_P2P: dict[tuple, object] = {}


def ensure_p2p_groups(prog: Program, comm: DistComm):
    """One 2-process NCCL group per *directed* pair of pipeline ranks (and position in the stage) that the
    program transfers between.  All point-to-point operations of one communicator run in issue order on one
    stream, so with a single communicator a receive posted ahead of time (say, of a gradient that arrives much
    later) would hold back every send issued after it; with a communicator per direction the only operations
    that queue behind each other are those that are ordered anyway.  Collective: same order on every process."""
    if not comm.cuda:
        return
    pairs = sorted({(ins.rank, ins.dst) for ins in prog.instrs if isinstance(ins, Transfer)})
    n_pos = comm.mesh.unstack[0].size
    from ..utils import config

    if config.p2p_backend.value == "native":
        from .p2p_native import NcclP2P

        procs = [(comm.mesh.unstack[src].flat_devices[pos].process_index, comm.mesh.unstack[dst].flat_devices[pos].process_index)
                 for src, dst in pairs for pos in range(n_pos)]
        key = comm.mesh._key()
        if key not in _NATIVE_P2P:
            _NATIVE_P2P[key] = NcclP2P(procs, comm.device)
        else:
            _NATIVE_P2P[key].add_pairs(procs)
        comm.native_p2p = _NATIVE_P2P[key]
        return
    mesh_key = comm.mesh._key()
    for src, dst in pairs:
        if (src, dst) in comm.p2p_groups:
            continue
        if (mesh_key, src, dst) in _P2P_GROUPS:  # made for another compiled function on the same mesh
            comm.p2p_groups[(src, dst)] = _P2P_GROUPS[(mesh_key, src, dst)]
            continue
        mine = None
        for pos in range(n_pos):
            procs = [comm.mesh.unstack[src].flat_devices[pos].process_index,
                     comm.mesh.unstack[dst].flat_devices[pos].process_index]
            g = dist.new_group(ranks=procs)
            if pos == comm.pos_in_stage and comm.rank in (src, dst):
                mine = g
        comm.p2p_groups[(src, dst)] = mine
        _P2P_GROUPS[(mesh_key, src, dst)] = mine


def ensure_groups(prog: Program, comm: DistComm):
    """Create, in program order and on every process, all process groups the program needs."""
    ensure_p2p_groups(prog, comm)
    seen = set()
    for ins in prog.instrs:
        ranks = getattr(ins, "ranks", None)
        if ranks is not None and tuple(ranks) not in seen:
            seen.add(tuple(ranks))
            comm._group(ranks)
