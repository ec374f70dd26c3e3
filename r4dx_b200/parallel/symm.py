"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

Allocation and the exchange of handles go through ``torch.distributed._symmetric_memory`` (CUDA
virtual memory + NVLink peer mappings); what the kernels get is a table of raw peer pointers.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch
import torch.distributed as dist


class SymmBuffer:
    """``nbytes`` of device memory on every rank, mapped into every rank's address space."""

    def __init__(self, nbytes: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group or dist.group.WORLD
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr or 0)
        except Exception:
            self.multicast_ptr = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def ptr_table(self, offset: int = 0):
        """ctypes array of ``world`` pointers, each ``offset`` bytes into that rank's buffer."""
        arr = (ctypes.c_void_p * self.world)()
        for i, p in enumerate(self.ptrs):
            arr[i] = p + offset
        return arr

    def local_view(self, offset: int, nbytes: int, dtype) -> torch.Tensor:
        return self.local[offset:offset + nbytes].view(dtype)
