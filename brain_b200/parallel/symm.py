"""Symmetric peer memory: one arena per rank, allocated and exchanged through
``torch.distributed._symmetric_memory`` (CUDA VMM handles over the process group's store), from
which the fused communication kernels get every peer's base pointer.  Sub-allocations are carved
at 256-byte aligned offsets, identical on every rank, so ``peer_ptrs(t)`` is base + offset."""
from __future__ import annotations

import math
from typing import List

import torch
import torch.distributed as dist


def default_wait_seconds() -> float:
    """Limit of every in-kernel wait on a peer (a flag another GPU writes).  Ranks meet at these
    waits after identical work, so steady-state skew is milliseconds; 2 s covers first-step set-up
    skew while keeping a shared GPU from being held by a rank whose peer has gone.
    ``BRAIN_PEER_WAIT_S`` overrides it."""
    import os
    return float(os.environ.get("BRAIN_PEER_WAIT_S", "2.0"))


class SymmArena:
    def __init__(self, nbytes: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.base_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.cursor = 0
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = numel * esz
        off = (self.cursor + 255) // 256 * 256
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted: need {off + nbytes}, have {self.nbytes}")
        self.cursor = off + nbytes
        return self.buf[off:off + nbytes].view(dtype)

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.buf.data_ptr()
        assert 0 <= off < self.nbytes, "tensor is not inside this arena"
        return off

    def peer_ptrs(self, t: torch.Tensor) -> List[int]:
        off = self.offset_of(t)
        return [b + off for b in self.base_ptrs]

    def multicast_ptr(self, t: torch.Tensor) -> int:
        """NVLS multicast address of ``t`` (0 when the fabric has no multicast support)."""
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        return mc + self.offset_of(t) if mc else 0
