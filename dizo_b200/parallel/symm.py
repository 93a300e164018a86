"""Symmetric (peer-visible) device memory for the fused collectives.

Every rank allocates the same region with ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exchanged over the process group; NVSwitch multicast mapping when the platform has
it) and learns every peer's base pointer.  A :class:`SymmRegion` hands out equally laid-out
sub-buffers: the local tensor view plus a device array with the peers' pointers to the same
sub-buffer, which is what the kernels in ``csrc/comm_*.cu`` take.  Flag words live in the same
region and are zero-initialised before first use; epochs only grow.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class SymmRegion:
    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        nbytes = (nbytes + 255) // 256 * 256
        self.nbytes = nbytes
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buf, group=self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr)
        except Exception:
            self.multicast_ptr = 0
        from ..ops import _lib
        for p in self.ptrs:                       # checked-store build: the peers' regions are writable
            _lib.note_range(p, nbytes)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self._cursor = 0

    def alloc(self, nbytes: int, align: int = 256):
        """-> (byte offset, local uint8 view, device int64 array of the peers' pointers)."""
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric region exhausted ({off + nbytes} > {self.nbytes} bytes)")
        self._cursor = off + nbytes
        view = self.buf[off:off + nbytes]
        ptrs = torch.tensor([p + off for p in self.ptrs], dtype=torch.int64, device=self.device)
        return off, view, ptrs

    def alloc_tensor(self, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        esz = torch.empty(0, dtype=dtype).element_size()
        off, view, ptrs = self.alloc(n * esz)
        return view.view(dtype).view(*shape), ptrs, off

    def multicast_addr(self, off: int) -> int:
        return self.multicast_ptr + off if self.multicast_ptr else 0
