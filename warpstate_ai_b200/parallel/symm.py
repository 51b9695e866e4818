"""Symmetric memory: buffers that every rank of a single-node job can address directly.

A `SymmetricBuffer` is a CUDA tensor allocated from memory that all ranks map (CUDA VMM
allocations exchanged between the processes), plus the table of peer addresses *as seen from
this process* and, when the NVSwitch fabric offers it, a multimem address whose loads reduce
and whose stores broadcast inside the switch (NVLS).

The allocation and handle exchange use PyTorch's symmetric-memory allocator
(`torch.distributed._symmetric_memory`) over the existing process group; everything that touches
the memory afterwards is this package's own kernels (`ops/csrc/comm.cu`).  Kernels that read a
peer's memory use plain loads/stores or `multimem` instructions only.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class SymmetricBuffer:
    tensor: torch.Tensor          # this rank's buffer
    peer_ptrs: list[int]          # device addresses of every rank's buffer in this process
    multicast_ptr: int            # multimem address or 0
    rank: int
    world: int
    handle: object = None

    def barrier(self) -> None:
        if self.handle is not None:
            self.handle.barrier()


def nvls_allowed() -> bool:
    """NVLS (multimem) is used unless disabled; failure-handling tests turn it off."""
    return os.environ.get("WARPSTATE_NVLS", "1") != "0" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"


def allocate(numel: int, dtype: torch.dtype, device: torch.device, group=None) -> SymmetricBuffer:
    import torch.distributed._symmetric_memory as symm_mem

    group = group if group is not None else dist.group.WORLD
    name = group.group_name
    try:
        if not symm_mem.is_symm_mem_enabled_for_group(name):
            symm_mem.enable_symm_mem_for_group(name)
    except Exception:
        pass
    tensor = symm_mem.empty(numel, dtype=dtype, device=device)
    tensor.zero_()
    handle = symm_mem.rendezvous(tensor, group=name)
    ptrs = [int(p) for p in handle.buffer_ptrs]
    mc = int(getattr(handle, "multicast_ptr", 0) or 0) if nvls_allowed() else 0
    return SymmetricBuffer(tensor, ptrs, mc, handle.rank, handle.world_size, handle)
