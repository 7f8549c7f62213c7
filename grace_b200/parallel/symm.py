"""Symmetric heap: the memory every rank can address on every other rank.

Each rank owns one device allocation; the IPC handles are exchanged once
through the process group and every peer's region is mapped locally, so a
kernel running on rank ``r`` reads ``heap[p] + offset`` for any ``p`` with plain
loads over NVLink.  Offsets come from a bump allocator that every rank drives
with the same sequence of requests, hence they are identical everywhere.

``SymmetricHeap.virtual(W)`` builds W heaps inside ONE process on one GPU.  The
kernels then run once per virtual rank, phase by phase (all ranks compress and
publish, then all ranks exchange), which exercises the same protocol and code
without ever having two kernels wait on each other.

The reference has no such layer: its ranks meet only inside NCCL / Gloo /
Horovod calls (``grace_dl/dist/communicator/*.py``).
"""
from __future__ import annotations

import weakref
from typing import List, Optional

import torch
from torch import distributed as dist

from ..ops import native

_DT_CODE = {
    torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int8: "|i1",
    torch.int64: "<i8", torch.float16: "<f2", torch.float64: "<f8",
}


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier for a raw device pointer."""

    def __init__(self, ptr: int, numel: int, dtype: torch.dtype, owner):
        self._owner = owner
        self.__cuda_array_interface__ = {
            "shape": (numel,), "typestr": _DT_CODE[dtype], "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_ptr(ptr: int, numel: int, dtype: torch.dtype, device, owner=None) -> torch.Tensor:
    if numel == 0:
        return torch.empty(0, dtype=dtype, device=device)
    return torch.as_tensor(_RawCuda(ptr, numel, dtype, owner), device=device)


class SymmetricHeap:
    ALIGN = 256

    def __init__(self, nbytes: int, rank: int, world: int, device: torch.device, bases: List[int], owned: List[int],
                 imported: List[int]):
        self.nbytes = nbytes
        self.rank = rank
        self.world = world
        self.device = device
        self.bases = bases          # base pointer of every rank's heap as mapped in this process
        self._owned = owned         # pointers to cudaFree at close
        self._imported = imported   # pointers to unmap at close
        self._cursor = 0
        self._closed = False
        self._finalizer = weakref.finalize(self, SymmetricHeap._release, list(owned), list(imported))

    # -- construction -----------------------------------------------------
    @classmethod
    def create(cls, nbytes: int, group=None, device: Optional[torch.device] = None) -> "SymmetricHeap":
        """One heap per process of ``group`` (default group when None)."""
        C = native()
        device = torch.device(device if device is not None else torch.cuda.current_device())
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        nbytes = (nbytes + cls.ALIGN - 1) // cls.ALIGN * cls.ALIGN
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        with torch.cuda.device(device):
            base = C.heap_alloc(nbytes)
            if world == 1:
                return cls(nbytes, 0, 1, device, [base], [base], [])
            handle = C.heap_export(base)
            gathered: List[Optional[tuple]] = [None] * world
            dist.all_gather_object(gathered, (handle, device.index), group=group)
            bases, imported = [], []
            for r, (h, dev_index) in enumerate(gathered):
                if r == rank:
                    bases.append(base)
                else:
                    C.enable_peer_access(dev_index)
                    p = C.heap_import(h)
                    bases.append(p)
                    imported.append(p)
            dist.barrier(group=group)
        return cls(nbytes, rank, world, device, bases, [base], imported)

    @classmethod
    def virtual(cls, nbytes: int, world: int, device: Optional[torch.device] = None) -> List["SymmetricHeap"]:
        """``world`` heaps in this process: one object per virtual rank."""
        C = native()
        device = torch.device(device if device is not None else torch.cuda.current_device())
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        nbytes = (nbytes + cls.ALIGN - 1) // cls.ALIGN * cls.ALIGN
        with torch.cuda.device(device):
            bases = [C.heap_alloc(nbytes) for _ in range(world)]
        heaps = []
        for r in range(world):
            heaps.append(cls(nbytes, r, world, device, list(bases), [bases[r]], []))
        return heaps

    @classmethod
    def local(cls, nbytes: int, device: Optional[torch.device] = None) -> "SymmetricHeap":
        """Single-rank heap backed by the caching allocator (no IPC); used by
        the stand-alone compress ops."""
        device = torch.device(device if device is not None else torch.cuda.current_device())
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        nbytes = (nbytes + cls.ALIGN - 1) // cls.ALIGN * cls.ALIGN
        backing = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        heap = cls(nbytes, 0, 1, device, [backing.data_ptr()], [], [])
        heap._backing = backing
        return heap

    # -- allocation -------------------------------------------------------
    def alloc(self, nbytes: int) -> int:
        """Reserve ``nbytes`` and return the offset (same on every rank)."""
        off = (self._cursor + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if off + nbytes > self.nbytes:
            raise MemoryError("symmetric heap exhausted: need %d bytes at offset %d of %d" % (nbytes, off, self.nbytes))
        self._cursor = off + nbytes
        return off

    def view(self, offset: int, numel: int, dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        """Tensor over heap memory of ``rank`` (default: this rank)."""
        r = self.rank if rank is None else rank
        return tensor_from_ptr(self.bases[r] + offset, numel, dtype, self.device, owner=self)

    @property
    def free_bytes(self) -> int:
        return self.nbytes - self._cursor

    def carve(self, nbytes: int) -> "SymmetricHeap":
        """Sub-heap of ``nbytes`` inside this heap: same mappings, own bump allocator, frees nothing.

        Every rank must carve in the same order (the offset is part of the address every peer computes).
        Raises ``MemoryError`` when the parent has no room left."""
        nbytes = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        off = self.alloc(nbytes)
        child = SymmetricHeap(nbytes, self.rank, self.world, self.device, [b + off for b in self.bases], [], [])
        child._parent = self          # keeps the mapping alive for as long as the child is in use
        return child

    # -- teardown ---------------------------------------------------------
    @staticmethod
    def _release(owned, imported):
        try:
            C = native()
            for p in imported:
                C.heap_release(p)
            for p in owned:
                C.heap_free(p)
        except Exception:
            pass

    def close(self):
        """Unmap the peers' regions and free this rank's region now (all kernels using the heap must
        have finished on every rank: synchronise and barrier first)."""
        if not self._closed:
            self._closed = True
            self._finalizer()
