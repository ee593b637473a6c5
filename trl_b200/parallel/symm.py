"""Symmetric memory arenas: buffers that every rank of the node maps, so kernels can ld/st (or
multimem.*) peer memory directly.

Allocation, handle exchange and mapping are done by ``torch.distributed._symmetric_memory`` (plumbing);
everything that moves data is in ``csrc/comm.cu``.  An arena is one large symmetric allocation from
which the engine carves its flat parameter / gradient buckets, so peer addresses are
``peer_base[p] + offset`` and one rendezvous serves all buckets.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as td

from . import dist as D


class SymmArena:
    def __init__(self, nbytes: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else td.group.WORLD
        nbytes = (nbytes + 255) // 256 * 256
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.pad_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.nbytes = nbytes
        self._cursor = 0
        self.buf.zero_()
        torch.cuda.synchronize()
        td.barrier(group=self.group)

    def carve(self, numel: int, dtype: torch.dtype) -> tuple[torch.Tensor, int]:
        """Returns (tensor view, byte offset inside the arena); 256-byte aligned."""
        esz = torch.empty(0, dtype=dtype).element_size()
        off = (self._cursor + 255) // 256 * 256
        end = off + numel * esz
        if end > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted ({end} > {self.nbytes} bytes)")
        self._cursor = end
        return self.buf[off:end].view(dtype), off

    def peers(self, byte_offset: int = 0):
        """ctypes uint64[world] of every rank's address of ``arena + byte_offset``."""
        return (ctypes.c_ulonglong * self.world)(*[p + byte_offset for p in self.peer_ptrs])

    def pads(self):
        return (ctypes.c_ulonglong * self.world)(*self.pad_ptrs)

    def mc(self, byte_offset: int = 0):
        return ctypes.c_void_p(self.multicast_ptr + byte_offset) if self.multicast_ptr else None


class SyncWords:
    """Device words a comm kernel family shares: epoch counter + local gate/arrival counter.  One
    instance per (channel, stream of use); all ranks must launch the same kernel sequence on it."""

    def __init__(self, device, channel: int):
        self.words = torch.zeros(4, dtype=torch.int32, device=device)
        self.channel = channel

    @property
    def epoch_ptr(self):
        return ctypes.c_void_p(self.words.data_ptr())

    @property
    def gate_ptr(self):
        return ctypes.c_void_p(self.words.data_ptr() + 4)


def symmetric_available() -> bool:
    if not (D.is_initialized() and torch.cuda.is_available() and D.world_size() > 1):
        return False
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
        return True
    except Exception:
        return False
