"""Peer-mapped ("symmetric") device memory and the flag arrays the NVLink kernels use.

Every rank allocates a buffer of the same size; after the rendezvous each rank holds the
device addresses of all ranks' buffers, so kernels can issue plain loads/stores on peer
memory over NVLink.  Allocation and handle exchange use torch's symmetric-memory
allocator (CUDA VMM + fd passing over the process group's store); everything that
touches the memory afterwards is this package's own kernels.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K

MAX_RANKS = 8


def ptr_array(ptrs: List[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class SymmBuffer:
    """A tensor whose storage is mapped on every rank of ``group``."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, zero: bool = True):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks per NVLink domain")
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        if zero:
            self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        assert self.ptrs[self.rank] == self.tensor.data_ptr()
        # NVSwitch multicast mapping of the same buffers (0 when the fabric or the driver
        # has no NVLS support): the target of this package's multimem.ld_reduce / multimem.st
        self.multicast_ptr: int = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        # MB200_NVLS: "0" never, "1" whenever there is a mapping, unset: from 4 ranks up.
        # With two ranks a rank reads one peer either way and the trip through the switch's
        # reduction unit only adds latency (256 MiB all-reduce: 645 GB/s on plain peer loads,
        # 379 GB/s through multimem); with four the in-switch sum wins (649 against 613).
        nvls = os.environ.get("MB200_NVLS", "auto")
        if nvls == "0" or (nvls != "1" and self.world < 4):
            self.multicast_ptr = 0
        self._elt = self.tensor.element_size()
        self._ptr_arrays: dict = {}
        nbytes = numel * self._elt
        for p in self.ptrs:                     # checked builds: the ranges kernels may touch
            K.bounds_register(p, nbytes, device)
        if self.multicast_ptr:
            K.bounds_register(self.multicast_ptr, nbytes, device)

    def ptrs_at(self, elem_offset: int):
        """ctypes array of every rank's address of element ``elem_offset``."""
        arr = self._ptr_arrays.get(elem_offset)
        if arr is None:       # trainers ask for the same few offsets (buckets, units) every step
            off = elem_offset * self._elt
            arr = ptr_array([p + off for p in self.ptrs])
            if len(self._ptr_arrays) < 4096:
                self._ptr_arrays[elem_offset] = arr
        return arr

    def mc_at(self, elem_offset: int) -> Optional[int]:
        """Multicast address of element ``elem_offset`` (None without NVLS): a
        ``multimem.ld_reduce`` there returns the sum over all ranks' copies, a
        ``multimem.st`` writes all of them."""
        if not self.multicast_ptr:
            return None
        return self.multicast_ptr + elem_offset * self._elt

    def peer_view(self, rank: int, numel: int, offset: int = 0) -> torch.Tensor:
        return self.handle.get_buffer(rank, (numel,), self.tensor.dtype, offset)


class FlagArray:
    """Per-rank array of epoch flags: ``flags[slot * MAX_RANKS + source_rank]``."""

    def __init__(self, n_slots: int, device: torch.device, group=None):
        self.n_slots = n_slots
        self.buf = SymmBuffer(n_slots * MAX_RANKS, torch.int32, device, group)
        self.rank, self.world = self.buf.rank, self.buf.world
        self.ptrs = ptr_array(self.buf.ptrs)
        self.my_ptr = self.buf.ptrs[self.rank]
        self.counter = torch.zeros(8, dtype=torch.int32, device=device)
        self._barrier_epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group or dist.group.WORLD)

    def barrier(self, slot: int) -> None:
        """Device-side flag barrier on the current stream (bounded wait)."""
        self._barrier_epoch += 1
        K.check(K.lib().mb200_barrier(self.ptrs, self.rank, self.world, slot,
                                      self._barrier_epoch,
                                      K.status_word(self.buf.tensor.device).data_ptr(),
                                      K.stream_ptr()), "barrier")
