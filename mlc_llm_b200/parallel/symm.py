"""Symmetric peer buffers: the same allocation on every rank of a group, each rank holding device
pointers to all peers' copies (NVLink peer access through NVSwitch).

Backed by ``torch.distributed._symmetric_memory`` (``cuMemCreate`` + handle exchange over the
process group's store; no NVSHMEM needed).  The reference's counterpart is the NVSHMEM heap its
disaggregation path allocates (``cpp/serve/engine.cc:410-425``) and the CUDA-IPC buffers of its
custom all-reduce (``compiler_pass/pipeline.py:185-189``).

Only plain loads / stores / reductions from kernels of this package touch peer pointers; peer
memory is never handed to library kernels and never read through TMA.
"""

from __future__ import annotations

import os
from typing import List

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """``nbytes`` of zero-initialised device memory on every rank of ``group``."""

    def __init__(self, nbytes: int, group=None, device: torch.device = None):
        import torch.distributed._symmetric_memory as symm_mem  # pylint: disable=import-outside-toplevel

        group = group if group is not None else dist.group.WORLD
        device = device or torch.device("cuda", torch.cuda.current_device())
        nbytes = (int(nbytes) + 255) & ~255
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, group)
        self.rank = int(self.handle.rank)
        self.world_size = int(self.handle.world_size)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        # multicast address of the allocation (NVLS: one load / store / reduction reaches every rank's
        # copy inside the NVSwitch); 0 when the fabric or the driver offers none
        self.mc_ptr = 0
        if os.environ.get("MLCB_MULTIMEM", "1") != "0":
            try:
                self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            except Exception:  # pylint: disable=broad-except
                self.mc_ptr = 0
        self.nbytes = nbytes
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def peer_ptr(self, rank: int, offset: int = 0) -> int:
        return self.ptrs[rank] + offset

    def view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """Typed view of this rank's copy."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset: offset + nbytes].view(dtype).view(*shape)


class LocalBuffer:
    """Single-process stand-in with the same interface (world size 1; also used on one GPU to run
    the fused kernels in their degenerate form)."""

    def __init__(self, nbytes: int, device: torch.device):
        nbytes = (int(nbytes) + 255) & ~255
        self.local = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.rank, self.world_size = 0, 1
        self.ptrs = [self.local.data_ptr()]
        self.mc_ptr = 0
        self.nbytes = nbytes

    peer_ptr = SymmetricBuffer.peer_ptr
    view = SymmetricBuffer.view
