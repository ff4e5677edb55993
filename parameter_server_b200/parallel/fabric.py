"""Symmetric heap over NVLink: the transport of the device data plane.

Every rank process owns one heap (a single ``cudaMalloc``) on its GPU, exports
it with CUDA IPC and maps every peer's heap. Fused kernels then read and write
peer memory directly; ordering is by release/acquire flag words inside the
heaps. This replaces the reference's socket transport
(``system/van.cc:27-269``) for everything that is not control traffic.

Three ways to build one:

* :meth:`Fabric.from_process_group` -- one rank per GPU (``torchrun``), handles
  exchanged through ``torch.distributed``;
* :meth:`Fabric.single` -- one rank, no peers;
* :meth:`Fabric.emulated` -- ``S`` heaps on ONE GPU inside one process, so the
  multi-shard kernels can be exercised on a single device. Kernels of different
  virtual ranks are then launched one after another on one stream (never
  concurrently, since one of them may wait on a flag another one sets).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np
import torch

from ..ops import _lib

_TORCH2NP = {
    torch.float32: "<f4", torch.float64: "<f8", torch.int32: "<i4", torch.int64: "<i8",
    torch.uint8: "|u1", torch.int8: "|i1", torch.float16: "<f2", torch.int16: "<i2",
    torch.uint32: "<u4", torch.uint64: "<u8",
}


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier for a raw device address."""

    def __init__(self, address: int, shape, typestr: str, owner):
        self.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": typestr, "data": (address, False), "version": 2,
        }
        self._owner = owner


class Fabric:
    def __init__(self, rank: int, world: int, device: torch.device, heap_bytes: int,
                 bases: List[int], owned: List[int], opened: List[int], group=None):
        self.rank, self.world, self.device = rank, world, device
        self.heap_bytes = heap_bytes
        self.bases = bases            # base address of every rank's heap in THIS process
        self._owned = owned           # heaps this object must cudaFree
        self._opened = opened         # IPC mappings this object must close
        self.group = group
        self._closed = False

    # ---------------------------------------------------------------- constructors
    @staticmethod
    def _alloc(nbytes: int) -> int:
        p = C.c_void_p()
        _lib.check(_lib.lib().psb_heap_alloc(C.byref(p), nbytes), "heap alloc", kernels=0)
        return p.value

    @classmethod
    def single(cls, heap_bytes: int, device=None) -> "Fabric":
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(device):
            base = cls._alloc(heap_bytes)
        return cls(0, 1, device, heap_bytes, [base], [base], [])

    @classmethod
    def emulated(cls, world: int, heap_bytes: int, device=None) -> List["Fabric"]:
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(device):
            bases = [cls._alloc(heap_bytes) for _ in range(world)]
        fabs = [cls(r, world, device, heap_bytes, bases, [bases[r]], []) for r in range(world)]
        return fabs

    @classmethod
    def from_process_group(cls, heap_bytes: int, group=None) -> "Fabric":
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        device = torch.device("cuda", torch.cuda.current_device())
        L = _lib.lib()
        base = cls._alloc(heap_bytes)
        nb = L.psb_ipc_handle_bytes()
        buf = C.create_string_buffer(nb)
        _lib.check(L.psb_ipc_export(base, buf), "ipc export", kernels=0)
        mine = (rank, torch.cuda.current_device(), bytes(buf.raw))
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        bases, opened = [0] * world, []
        for r, dev, handle in everyone:
            if r == rank:
                bases[r] = base
                continue
            p = C.c_void_p()
            hb = C.create_string_buffer(handle, nb)
            _lib.check(L.psb_ipc_open(hb, C.byref(p)), f"ipc open rank {r}", kernels=0)
            bases[r] = p.value
            opened.append(p.value)
        dist.barrier(group=group)
        return cls(rank, world, device, heap_bytes, bases, [base], opened, group)

    # ---------------------------------------------------------------- access
    def ptr(self, rank: int, offset: int = 0) -> int:
        assert 0 <= offset <= self.heap_bytes
        return self.bases[rank] + offset

    def view(self, offset: int, shape, dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        """A tensor aliasing heap memory. Only heaps that live on this process's
        device may be viewed (the local heap, or any heap of an emulated fabric);
        peer heaps are reached from kernels through :meth:`ptr`."""
        rank = self.rank if rank is None else rank
        if dtype == torch.bfloat16:     # no array-interface code for bf16: alias as int16 and reinterpret
            return self.view(offset, shape, torch.int16, rank).view(torch.bfloat16)
        n = int(np.prod(shape)) if len(shape) else 1
        assert offset + n * torch.empty((), dtype=dtype).element_size() <= self.heap_bytes
        raw = _RawCuda(self.bases[rank] + offset, shape, _TORCH2NP[dtype], self)
        return torch.as_tensor(raw, device=self.device)

    def barrier(self):
        if self.group is not None or (self.world > 1 and self._opened):
            import torch.distributed as dist
            dist.barrier(group=self.group)

    def close(self):
        if self._closed:
            return
        self._closed = True
        L = _lib.lib()
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            L.psb_ipc_close(p)
        if self._opened:
            self.barrier()
        for p in self._owned:
            L.psb_heap_free(p)


class HeapLayout:
    """Bump allocator for offsets inside a symmetric heap; identical on every
    rank, so ``offset`` addresses the same object in every heap."""

    def __init__(self, align: int = 256):
        self.align = align
        self.size = 0
        self.items = {}

    def add(self, name: str, nbytes: int) -> int:
        off = (self.size + self.align - 1) // self.align * self.align
        self.items[name] = (off, nbytes)
        self.size = off + nbytes
        return off

    def __getitem__(self, name: str) -> int:
        return self.items[name][0]

    def total(self) -> int:
        return (self.size + self.align - 1) // self.align * self.align
