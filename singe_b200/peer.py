"""Peer-mapped device buffers of a tensor-parallel group, for the fused all-reduce of the decode step.

Every rank allocates its buffers with ``singe_peer_buffer_create`` (plain ``cudaMalloc`` memory plus a CUDA IPC
handle), the handles travel through ``torch.distributed`` (``all_gather_object``, i.e. the host-side bootstrap the
process group already has), and every rank opens the other ranks' buffers.  What comes out is, per buffer, the list
of ``world`` device pointers ``singe_allreduce_add_rms_norm_bf16`` takes.  torch is plumbing here: rendezvous only.

Replaces nothing in the reference directly: singe-nccl registers communicator buffers through NCCL
(singe-nccl/src/communicator/mod.rs); this is the peer-memory counterpart the fused kernel needs.
"""
from __future__ import annotations

import ctypes

from . import kernel_sys as ks

HANDLE_BYTES = 64


class PeerBuffer:
    """One symmetric buffer: ``pointers[r]`` is rank r's copy as mapped into this process."""

    def __init__(self, group, rank: int, world: int, nbytes: int):
        lib = ks.lib()
        self.rank, self.world, self.nbytes = rank, world, nbytes
        local = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(HANDLE_BYTES)
        code = lib.singe_peer_buffer_create(nbytes, ctypes.byref(local), handle)
        if code != ks.OK:
            raise RuntimeError(f"peer buffer create: status {code} ({ks.status_string(code)})")
        self.local = local.value
        handles = [None] * world
        group.all_gather_object(handles, bytes(handle.raw))
        self.pointers = []
        self._opened = []
        for r in range(world):
            if r == rank:
                self.pointers.append(self.local)
                continue
            remote = ctypes.c_void_p()
            code = lib.singe_peer_buffer_open(ctypes.create_string_buffer(handles[r], HANDLE_BYTES),
                                              ctypes.byref(remote))
            if code != ks.OK:
                raise RuntimeError(f"peer buffer open (rank {r}): status {code} ({ks.status_string(code)})")
            self.pointers.append(remote.value)
            self._opened.append(remote.value)
        self.array = (ctypes.c_void_p * world)(*self.pointers)  # the host array of device pointers the C ABI takes
        group.barrier()  # every rank has mapped every buffer before anyone uses them

    def close(self, group) -> None:
        """Unmaps the peers' buffers, then (after a barrier) frees the local one."""
        lib = ks.lib()
        for pointer in self._opened:
            lib.singe_peer_buffer_close(pointer)
        self._opened = []
        group.barrier()
        if self.local:
            lib.singe_peer_buffer_destroy(self.local)
            self.local = 0


class TwoPhaseAllReduce:
    """Buffers of the two-phase collective (``singe_allreduce_two_phase_add_rms_norm_bf16``): the packet buffer the
    peers push their partial rows into, the packet buffer every owner pushes its normalised rows into, and the local
    epoch state.  The GEMMs write their partial sums into ordinary local memory (``partial_pointer(which)``) and the
    normalised rows come out in an ordinary local tensor."""

    def __init__(self, group, rank: int, world: int, rows: int, width: int, wait_limit_kcycles: int = 0,
                 replicated: bool = False):
        import torch

        if world > 8:
            raise ValueError("the fused all-reduce serves one NVSwitch domain: at most 8 ranks")
        self.group, self.rank, self.world, self.rows, self.width = group, rank, world, rows, width
        # replicated: every rank receives every partial row and reduces all rows itself (one NVLink trip, for two ranks)
        self.replicated = replicated
        self.rpr = rows if replicated else (rows + world - 1) // world
        self.receive = PeerBuffer(group, rank, world, world * self.rpr * width * 4)
        # packets of all normalised rows, then this rank's staging area for the rows it owns
        self.gather = self.receive if replicated else PeerBuffer(group, rank, world, (rows + self.rpr) * width * 4)
        self.state = torch.zeros(4, dtype=torch.int32, device="cuda")
        if wait_limit_kcycles:
            self.state[2] = wait_limit_kcycles
        self.partials = [torch.empty((rows, width), dtype=torch.bfloat16, device="cuda") for _ in range(2)]

    def partial_pointer(self, which: int) -> int:
        return self.partials[which].data_ptr()

    def reduce_add_norm(self, stream: int, which: int, hidden: int, normed: int, weight: int, eps: float,
                        status: int) -> None:
        code = ks.lib().singe_allreduce_two_phase_add_rms_norm_bf16(
            stream, hidden, normed, weight, self.partials[which].data_ptr(), self.receive.array, self.gather.array,
            self.state.data_ptr(), self.rank, self.world, self.rows, self.width, eps, int(self.replicated), status)
        if code != ks.OK:
            raise RuntimeError(f"two-phase all-reduce: status {code} ({ks.status_string(code)})")

    def close(self) -> None:
        for buffer in ((self.receive,) if self.replicated else (self.receive, self.gather)):
            buffer.close(self.group)


class PeerAllReduce:
    """The buffers one decode step needs: two partial buffers [rows, width] bf16 that alternate between the
    o_proj and down_proj collectives, the flag arrays, and the local epoch state."""

    def __init__(self, group, rank: int, world: int, rows: int, width: int):
        if world > 8:
            raise ValueError("the fused all-reduce serves one NVSwitch domain: at most 8 ranks")
        self.group, self.rank, self.world, self.rows, self.width = group, rank, world, rows, width
        self.partials = [PeerBuffer(group, rank, world, rows * width * 2) for _ in range(2)]
        self.flags = PeerBuffer(group, rank, world, 256)      # uint32[world], padded
        self.state = PeerBuffer(group, rank, world, 256)      # local use only: uint32[2]; peers never touch it

    def partial_pointer(self, which: int) -> int:
        """Where this rank's GEMM writes its partial rows for collective ``which`` (0: o_proj, 1: down_proj)."""
        return self.partials[which].local

    def reduce_add_norm(self, stream: int, which: int, hidden: int, normed: int, weight: int, eps: float,
                        status: int) -> None:
        code = ks.lib().singe_allreduce_add_rms_norm_bf16(
            stream, hidden, normed, weight, self.partials[which].array, self.flags.array, self.state.local, self.rank,
            self.world, self.rows, self.width, eps, status)
        if code != ks.OK:
            raise RuntimeError(f"fused all-reduce: status {code} ({ks.status_string(code)})")

    def close(self) -> None:
        for buffer in (*self.partials, self.flags, self.state):
            buffer.close(self.group)
