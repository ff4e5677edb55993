"""KVLayer on the GPUs: dense tensors keyed by layer id, pushed (summed over
workers, then an updater) and pulled over peer memory.

Same placement rule as the reference's ``KVLayer::Slice``
(``parameter/kv_layer.h:121-158``): a layer with fewer than ``partition_thr``
elements lives whole on server ``(id * 991) % n``; a larger one is split evenly by
element range over all servers.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Tuple

import torch

from ..ops import _lib
from ..ops._lib import MAX_SHARDS, check, ptr, stream_ptr
from ..parallel.fabric import Fabric, HeapLayout

_vp, _u32, _u64, _i32, _f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float


class _Push(C.Structure):
    _fields_ = [("S", _i32), ("ts1", _u32), ("data", _vp), ("seg_begin", _u64 * (MAX_SHARDS + 1)),
                ("inbox", _vp * MAX_SHARDS), ("ready", _vp * MAX_SHARDS), ("done", _vp)]


class _Apply(C.Structure):
    _fields_ = [("S", _i32), ("ts1", _u32), ("updater", _i32), ("lr", _f32), ("n", _u64), ("data", _vp),
                ("inbox", _vp * MAX_SHARDS), ("ready", _vp * MAX_SHARDS), ("alive", C.c_uint8 * MAX_SHARDS),
                ("wait_iters", _u32), ("applied", _vp), ("done", _vp), ("status", _vp)]


class _Pull(C.Structure):
    _fields_ = [("S", _i32), ("need_applied", _u32), ("out", _vp), ("seg_begin", _u64 * (MAX_SHARDS + 1)),
                ("data", _vp * MAX_SHARDS), ("applied", _vp * MAX_SHARDS), ("wait_iters", _u32), ("status", _vp)]


def _declare():
    L = _lib.lib()
    if getattr(L, "_layer_declared", False):
        return L
    for name in ("psb_layer_push", "psb_layer_apply", "psb_layer_pull"):
        getattr(L, name).argtypes = [_vp, _vp]
    L.psb_layer_args_size.argtypes = [_i32]
    for i, st in enumerate((_Push, _Apply, _Pull)):
        if L.psb_layer_args_size(i) != C.sizeof(st):
            raise RuntimeError(f"{st.__name__}: binding is {C.sizeof(st)} bytes, library expects {L.psb_layer_args_size(i)}")
    L._layer_declared = True
    return L


UPDATERS = {"assign": 0, "add": 1, "sgd": 2}


class DeviceKVLayer:
    """All layers are declared up front (``layers``: {id: number of elements}) so
    that every rank computes the same heap layout."""

    def __init__(self, fabric: Fabric, layers: Dict[int, int], partition_thr: int = 1000, updater: str = "add",
                 lr: float = 0.1):
        self.L = _declare()
        self.fabric = fabric
        self.rank, self.S = fabric.rank, fabric.world
        self.updater, self.lr, self.thr = UPDATERS[updater], lr, partition_thr
        self.layers = dict(layers)
        lay = HeapLayout()
        self.meta = {}
        for i, (lid, n) in enumerate(sorted(layers.items())):
            seg = self.segments(lid, n)
            mx = max(seg[s + 1] - seg[s] for s in range(self.S))
            self.meta[lid] = dict(idx=i, n=n, seg=seg, cap=mx,
                                  data=lay.add(f"data{lid}", max(mx, 1) * 4),
                                  inbox=lay.add(f"inbox{lid}", self.S * max(mx, 1) * 4),
                                  flags=lay.add(f"flags{lid}", 4 * (self.S + 2)), ts=0)
        self.lay = lay
        assert lay.total() <= fabric.heap_bytes, "heap too small"
        dev = fabric.device
        self.sync = torch.zeros(8, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    @staticmethod
    def heap_bytes(layers: Dict[int, int], world: int, partition_thr: int = 1000) -> int:
        total = 0
        for lid, n in layers.items():
            mx = n if n < partition_thr else (n + world - 1) // world + 1
            total += (mx * 4 + 256) * (world + 1) + 4 * (world + 2) + 512
        return total + 4096

    def segments(self, lid: int, n: int) -> List[int]:
        """Element boundaries of the shards for layer ``lid``."""
        S = self.S
        if n < self.thr:
            owner = (lid * 991) % S
            return [0 if s <= owner else n for s in range(S + 1)]
        return [n * s // S for s in range(S)] + [n]

    def _p(self, rank, off):
        return self.fabric.ptr(rank, off)

    def push(self, lid: int, data: torch.Tensor, stream=None) -> int:
        m = self.meta[lid]
        assert data.numel() == m["n"] and data.dtype == torch.float32 and data.is_contiguous()
        ts = m["ts"]
        a = _Push()
        a.S, a.ts1, a.data = self.S, ts + 1, ptr(data)
        for s in range(self.S + 1):
            a.seg_begin[s] = m["seg"][s]
        for s in range(self.S):
            a.inbox[s] = self._p(s, m["inbox"] + self.rank * max(m["cap"], 1) * 4)
            a.ready[s] = self._p(s, m["flags"] + 4 * (2 + self.rank))
        a.done = self.sync.data_ptr()
        check(self.L.psb_layer_push(C.byref(a), stream_ptr(stream)), "layer_push")
        return ts

    def apply(self, lid: int, alive=None, wait_iters: int = 0, stream=None):
        """Owner side of push round ``ts`` of this layer (every rank calls it)."""
        m = self.meta[lid]
        ts = m["ts"]
        m["ts"] += 1
        n = m["seg"][self.rank + 1] - m["seg"][self.rank]
        a = _Apply()
        a.S, a.ts1, a.updater, a.lr, a.n = self.S, ts + 1, self.updater, self.lr, n
        a.data = self._p(self.rank, m["data"])
        for r in range(self.S):
            a.inbox[r] = self._p(self.rank, m["inbox"] + r * max(m["cap"], 1) * 4)
            a.ready[r] = self._p(self.rank, m["flags"] + 4 * (2 + r))
            a.alive[r] = 1 if (alive is None or alive[r]) else 0
        a.wait_iters = wait_iters
        a.applied, a.done, a.status = self._p(self.rank, m["flags"]), self.sync.data_ptr() + 8, ptr(self.status)
        check(self.L.psb_layer_apply(C.byref(a), stream_ptr(stream)), "layer_apply")

    def pull(self, lid: int, out: torch.Tensor, wait_for_round: int = 0, stream=None):
        """Gather the layer from its owners into ``out``; waits until the owners
        have applied ``wait_for_round`` pushes."""
        m = self.meta[lid]
        assert out.numel() == m["n"] and out.dtype == torch.float32 and out.is_contiguous()
        a = _Pull()
        a.S, a.need_applied, a.out = self.S, wait_for_round, ptr(out)
        for s in range(self.S + 1):
            a.seg_begin[s] = m["seg"][s]
        for s in range(self.S):
            a.data[s] = self._p(s, m["data"])
            a.applied[s] = self._p(s, m["flags"])
        a.status = ptr(self.status)
        check(self.L.psb_layer_pull(C.byref(a), stream_ptr(stream)), "layer_pull")

    def segment(self, lid: int) -> torch.Tensor:
        """This rank's owned segment of the layer (a view of heap memory)."""
        m = self.meta[lid]
        n = m["seg"][self.rank + 1] - m["seg"][self.rank]
        return self.fabric.view(m["data"], (n,), torch.float32)

    def check_status(self, what="kv layer"):
        _lib.check_status(self.status, what)
