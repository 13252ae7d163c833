"""Native point-to-point backend: 2-rank NCCL communicators driven through the C ABI of ``csrc/p2p_nccl.cu``.

One communicator (and one CUDA stream) per *directed* pair of processes, created collectively from unique ids
exchanged once over the default process group; every transfer is one NCCL group of byte-typed sends or
receives on that pair's stream.  Equivalent of the reference's cupy NCCL backend (src/jaxpp/dime2.py:72-197),
selected with ``JAXPP_B200_P2P=native``; the default backend issues the same transfers through
``torch.distributed``.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch
import torch.distributed as dist

from ..ops import native


class JpbP2POp(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("bytes", ctypes.c_longlong), ("peer", ctypes.c_int), ("is_send", ctypes.c_int)]


def _lib():
    lib = native.load()
    lib.jpb_p2p_last_error.restype = ctypes.c_char_p
    lib.jpb_p2p_unique_id.argtypes = [ctypes.c_char_p]
    lib.jpb_p2p_comm_create.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]
    lib.jpb_p2p_comm_destroy.argtypes = [ctypes.c_void_p]
    lib.jpb_p2p_batch.argtypes = [ctypes.c_void_p, ctypes.POINTER(JpbP2POp), ctypes.c_int, ctypes.c_void_p]
    return lib


def _check(lib, rc: int, what: str):
    if rc != 0:
        raise native.NativeError(f"{what} failed ({rc}): {lib.jpb_p2p_last_error().decode(errors='replace')}")


class NcclP2P:
    """Communicators for a set of directed process pairs ``(src_proc, dst_proc)`` (global ranks)."""

    def __init__(self, pairs: Sequence[tuple[int, int]], device: torch.device):
        self.lib = _lib()
        if not self.lib.jpb_p2p_available():
            raise native.NativeError("NCCL is not loadable: " + self.lib.jpb_p2p_last_error().decode(errors="replace"))
        self.device = device
        self.me = dist.get_rank()
        self.comms: dict[tuple[int, int], int] = {}
        self.streams: dict[tuple[int, int], torch.cuda.Stream] = {}
        self.add_pairs(pairs)

    def add_pairs(self, pairs: Sequence[tuple[int, int]]):
        """Collective over all processes: every process passes the same list."""
        pairs = sorted(set(p for p in pairs if p not in self.comms and p[0] != p[1]))
        if not pairs:
            return
        # the source of each pair draws the id; one all-gather publishes all of them
        mine = {}
        for src, dst in pairs:
            if src == self.me:
                buf = ctypes.create_string_buffer(128)
                _check(self.lib, self.lib.jpb_p2p_unique_id(buf), "jpb_p2p_unique_id")
                mine[(src, dst)] = buf.raw
        gathered: list = [None] * dist.get_world_size()
        dist.all_gather_object(gathered, mine)
        ids = {k: v for d in gathered for k, v in d.items()}
        # same global order everywhere: communicator creation blocks until the partner arrives
        with torch.cuda.device(self.device):
            for src, dst in pairs:
                if self.me not in (src, dst):
                    continue
                comm = ctypes.c_void_p()
                rank_in_pair = 0 if self.me == src else 1
                _check(self.lib, self.lib.jpb_p2p_comm_create(ids[(src, dst)], 2, rank_in_pair, ctypes.byref(comm)),
                       "jpb_p2p_comm_create")
                self.comms[(src, dst)] = comm.value
                self.streams[(src, dst)] = torch.cuda.Stream(self.device)
                # NCCL sets up the connection of a pair inside the first send / recv, and that set-up blocks the
                # host until the partner issues the matching call.  Do it here, where both ends are at the same
                # place in the same order, so that later transfers can be issued in any interleaving.
                warm = torch.zeros(16, dtype=torch.uint8, device=self.device)
                self._batch((src, dst), [warm], is_send=self.me == src)
                self.streams[(src, dst)].synchronize()

    def _batch(self, pair, tensors: Sequence[torch.Tensor], is_send: bool):
        """Enqueue one NCCL group on the pair's stream (the caller orders that stream against producers)."""
        ops = (JpbP2POp * len(tensors))()
        peer = 1 if is_send else 0
        for i, t in enumerate(tensors):
            if not t.is_contiguous():
                raise native.NativeError("p2p payloads must be contiguous")
            ops[i].ptr, ops[i].bytes, ops[i].peer, ops[i].is_send = t.data_ptr(), t.numel() * t.element_size(), peer, int(is_send)
        stream = self.streams[pair]
        _check(self.lib, self.lib.jpb_p2p_batch(self.comms[pair], ops, len(tensors), stream.cuda_stream), "jpb_p2p_batch")

    def send(self, dst_proc: int, tensors: Sequence[torch.Tensor], after: torch.cuda.Event) -> torch.cuda.Event:
        pair = (self.me, dst_proc)
        stream = self.streams[pair]
        stream.wait_event(after)
        self._batch(pair, tensors, True)
        done = torch.cuda.Event()
        done.record(stream)
        for t in tensors:
            t.record_stream(stream)
        return done

    def recv(self, src_proc: int, buffers: Sequence[torch.Tensor], after: torch.cuda.Event) -> torch.cuda.Event:
        pair = (src_proc, self.me)
        stream = self.streams[pair]
        stream.wait_event(after)
        self._batch(pair, buffers, False)
        done = torch.cuda.Event()
        done.record(stream)
        for t in buffers:
            t.record_stream(stream)
        return done

    def close(self):
        torch.cuda.synchronize(self.device)
        for comm in self.comms.values():
            self.lib.jpb_p2p_comm_destroy(comm)
        self.comms.clear()
