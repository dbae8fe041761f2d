"""Symmetric NVLink-visible memory and the collectives that run on it.

A :class:`SymmetricArena` is one fp32 buffer allocated with the same size on every rank of a
process group (``torch.distributed._symmetric_memory`` does the allocation and the exchange of
handles); every rank can address every peer's copy.  The library's own kernels do the rest:
bounded-wait barriers, pull-reductions to an owner, push-broadcasts from an owner, and GEMM
epilogues that add tiles into a peer's buffer or replicate results to all peers
(asdl_b200/csrc/symm_collectives.cu, asdl_b200/csrc/umma_gemm.cuh).

Replaces the packed ``dist.reduce`` / ``dist.broadcast`` calls of the reference
(asdl/precondition/natural_gradient.py:603-757).
"""
from typing import List, Sequence, Tuple

import os

import torch
import torch.distributed as dist

from .. import ops

__all__ = ['SymmetricArena']

FLAG_WORDS = 256  # must match SYMM_FLAG_WORDS in csrc/symm_collectives.cu
_ALIGN = 64       # elements (256 bytes)


def _round_up(v, m):
    return (v + m - 1) // m * m


class SymmetricArena:
    """Bump allocator over one symmetric fp32 buffer.

    Every rank has to make the same sequence of ``alloc`` calls, so that a tensor has the same
    offset on all ranks.  ``ptr(rank, offset)`` is the device address of that offset in
    ``rank``'s copy, valid in this process.
    """

    #: wall-clock limit of every barrier wait in milliseconds; ranks drift apart by the length of
    #: their owner-local work (inverses) and by host stalls, which this has to cover
    barrier_wait_ms = 5000

    #: barrier slot of the kernels that run on the communication stream (slot 0 belongs to the main stream)
    COMM_SLOT = 1

    def __init__(self, numel: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device('cuda', torch.cuda.current_device()) if device is None else device
        self.capacity = _round_up(int(numel), _ALIGN)
        self.buffer = symm_mem.empty(FLAG_WORDS + self.capacity, dtype=torch.float32, device=self.device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.peer_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.peers_dev = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=self.device)
        # NVLS: the address under which the NVSwitch sees all ranks' copies at once (multimem.ld_reduce
        # / multimem.st in the kernels); 0 when the fabric or the allocator offers none.  Switched off
        # with ASDL_B200_MULTIMEM=0: a process that dies while its memory is bound to a multicast
        # object can fault its peers' GPUs, so runs that expect ranks to leave use plain peer accesses.
        self.multicast_ptr = 0
        if os.environ.get('ASDL_B200_MULTIMEM', '1') != '0':
            try:
                self.multicast_ptr = int(getattr(self.handle, 'multicast_ptr', 0) or 0)
            except Exception:
                self.multicast_ptr = 0
        self.buffer.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self._cursor = 0

    @classmethod
    def local_group(cls, numel: int, world: int, device=None) -> List['SymmetricArena']:
        """``world`` arenas on ONE GPU that address each other like ranks on different GPUs do.

        For exercising the pull / push / GEMM-epilogue kernels without a second GPU.  The kernels
        of different emulated ranks run one after the other on the same stream, so anything that
        waits for a peer cannot work: :meth:`barrier` raises on such arenas.
        """
        device = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
        capacity = _round_up(int(numel), _ALIGN)
        buffers = [torch.zeros(FLAG_WORDS + capacity, dtype=torch.float32, device=device) for _ in range(world)]
        ptrs = [b.data_ptr() for b in buffers]
        arenas = []
        for r in range(world):
            a = cls.__new__(cls)
            a.group, a.device, a.capacity, a.buffer, a.handle = None, device, capacity, buffers[r], None
            a.rank, a.world, a.peer_ptrs = r, world, list(ptrs)
            a.multicast_ptr = 0
            a.peers_dev = torch.tensor(ptrs, dtype=torch.int64, device=device)
            a._cursor = 0
            a._emulated = True
            arenas.append(a)
        return arenas

    # allocation --------------------------------------------------------------------------------
    def alloc(self, *shape) -> Tuple[int, torch.Tensor]:
        """(offset in elements from the start of the buffer, zero-initialised view)."""
        numel = 1
        for s in shape:
            numel *= int(s)
        start = self._cursor
        if start + numel > self.capacity:
            raise RuntimeError(f'symmetric arena exhausted: need {start + numel}, have {self.capacity}')
        self._cursor = _round_up(start + numel, _ALIGN)
        offset = FLAG_WORDS + start
        return offset, self.buffer[offset:offset + numel].view(*shape)

    def ptr(self, rank: int, offset: int) -> int:
        return self.peer_ptrs[rank] + 4 * offset

    def mc_ptr(self, offset: int) -> int:
        """Multicast address of ``offset`` (a store to it reaches every rank's copy); 0 without NVLS."""
        return self.multicast_ptr + 4 * offset if self.multicast_ptr else 0

    def segments(self, pairs: Sequence[Tuple[int, int]]) -> torch.Tensor:
        """Device table of (offset, numel rounded up to 4) rows for the segment kernels."""
        rows = [[int(o), _round_up(int(n), 4)] for o, n in pairs]
        return torch.tensor(rows, dtype=torch.int64, device=self.device).reshape(-1, 2)

    # collectives -------------------------------------------------------------------------------
    def barrier(self, slot: int = 0):
        """All ranks' work issued before the barrier (on the current stream) is complete and
        visible to all peers after it.  The wait is bounded; a timeout is reported through
        :func:`asdl_b200.ops.check_status`."""
        if getattr(self, '_emulated', False) and self.world > 1:
            raise RuntimeError('emulated ranks share one GPU and cannot wait for each other')
        ops.extension().symm_barrier(self.peers_dev, self.rank, self.world, slot, int(self.barrier_wait_ms))

    def reduce_segments(self, segs: torch.Tensor, scale: float):
        """local[seg] <- scale * sum over ranks of their [seg] (pull over NVLink; ``multimem.ld_reduce``
        through the switch where the buffer has a multicast mapping)."""
        ops.extension().symm_reduce_segments(self.peers_dev, self.rank, self.world, segs, float(scale),
                                             self.multicast_ptr)

    def bcast_segments(self, segs: torch.Tensor):
        """every peer's [seg] <- local[seg] (push over NVLink; one multimem.st per 16 bytes where the
        buffer has a multicast mapping, one store per peer otherwise)."""
        ops.extension().symm_bcast_segments(self.peers_dev, self.rank, self.world, segs, self.multicast_ptr)

    def bucket_reduce(self, segs: torch.Tensor, scale: float, blocks: int = 16):
        """One gradient bucket, one kernel: announce that this rank's part of the bucket is in place,
        wait (bounded) for all ranks, then ``local[seg] <- scale * sum over ranks of their [seg]`` for
        the listed segments (``multimem.ld_reduce`` through the switch where available).  Every rank
        calls it for every bucket, with an empty list if it owns nothing in it; meant for a
        communication stream (it uses its own barrier slot)."""
        if getattr(self, '_emulated', False) and self.world > 1:
            raise RuntimeError('emulated ranks share one GPU and cannot wait for each other')
        ops.extension().symm_bucket_reduce(self.peers_dev, self.rank, self.world, self.COMM_SLOT, segs, float(scale),
                                           self.multicast_ptr, int(self.barrier_wait_ms), int(blocks))

    def mirror_lower(self, mats: torch.Tensor, n_max: int):
        """For every row (offset, n) of ``mats``: the n x n matrix at ``offset`` of the local buffer
        gets its upper triangle from its lower one."""
        ops.extension().symm_mirror_lower(self.buffer, mats, int(n_max))

    def reduce_slots(self, table: torch.Tensor, slot_stride: int, n_max: int, beta: float):
        """For every row (factor offset, offset of slot 0, n) of ``table``: the local n x n factor
        becomes ``beta * factor + sum over ranks of its slots`` (lower triangles, mirrored); slot r
        lies ``r * slot_stride`` elements after slot 0.  Peers fill the slots with the stores of
        their SYRK epilogues; this reduction reads local memory only."""
        ops.extension().symm_reduce_slots(self.buffer, table, self.world, int(slot_stride), int(n_max), float(beta))

    def pull_slots(self, table: torch.Tensor, n_max: int, beta: float):
        """For every row (factor offset, contribution offset, n) of ``table``: the local n x n factor becomes
        ``beta * factor + sum over ranks of the n x n block at `contribution offset` of THAT rank's buffer``
        (lower triangles, mirrored).  Every rank's SYRK epilogue stores into its own buffer; the owner reads
        the peers' copies with coalesced loads over NVLink."""
        ops.extension().symm_pull_slots(self.buffer, self.peers_dev, table, self.world, int(n_max), float(beta))

    def scale_segments(self, segs: torch.Tensor, beta: float):
        ops.extension().symm_scale_segments(self.buffer, segs, float(beta))
