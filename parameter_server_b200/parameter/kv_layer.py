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
    _fields_ = [("S", _i32), ("ts1", _u32), ("need_applied", _u32), ("wait_iters", _u32), ("data", _vp),
                ("seg_begin", _u64 * (MAX_SHARDS + 1)), ("inbox", _vp * MAX_SHARDS), ("ready", _vp * MAX_SHARDS),
                ("applied", _vp * MAX_SHARDS), ("done", _vp), ("status", _vp)]


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
    L.psb_fabric_copy.argtypes = [_vp, _vp, _u64, _i32, _vp, _vp]
    for i, st in enumerate((_Push, _Apply, _Pull)):
        if L.psb_layer_args_size(i) != C.sizeof(st):
            raise RuntimeError(f"{st.__name__}: binding is {C.sizeof(st)} bytes, library expects {L.psb_layer_args_size(i)}")
    L._layer_declared = True
    return L


UPDATERS = {"assign": 0, "add": 1, "sgd": 2}


def _up4(x: int) -> int:
    return (x + 3) // 4 * 4


class DeviceKVLayer:
    """All layers are declared up front (``layers``: {id: number of elements}) so
    that every rank computes the same heap layout.

    Per layer the heap holds the owned segment, a ring of ``ring`` inbox slots per
    source (round ``t`` uses slot ``t % ring``) and the flag words: the owner's
    ``applied`` counter and one ``ready`` flag per (slot, source). A push of round
    ``t`` waits on the device, bounded, until every owner has applied round
    ``t - ring`` (the round that last used the slot), so a fast worker can run at
    most ``ring`` rounds ahead of a slow owner and never overwrites data that is
    still being summed. Arrival counters are per layer: layers may be pushed and
    applied on different streams.

    ``apply`` of a round waits on the device only for *other* ranks' pushes: this
    rank's own push of the round is ordered before it by a CUDA event (two kernels
    of one GPU never wait for one another on the device).
    """

    def __init__(self, fabric: Fabric, layers: Dict[int, int], partition_thr: int = 1000, updater: str = "add",
                 lr: float = 0.1, ring: int = 2):
        self.L = _declare()
        self.fabric = fabric
        self.rank, self.S = fabric.rank, fabric.world
        self.updater, self.lr, self.thr, self.ring = UPDATERS[updater], lr, partition_thr, max(1, ring)
        self.layers = dict(layers)
        lay = HeapLayout()
        self.meta = {}
        for i, (lid, n) in enumerate(sorted(layers.items())):
            seg = self.segments(lid, n)
            cap = max(4, _up4(max(seg[s + 1] - seg[s] for s in range(self.S))))
            self.meta[lid] = dict(idx=i, n=n, seg=seg, cap=cap,
                                  data=lay.add(f"data{lid}", cap * 4),
                                  inbox=lay.add(f"inbox{lid}", self.ring * self.S * cap * 4),
                                  flags=lay.add(f"flags{lid}", 4 * (1 + self.ring * self.S)),
                                  push_ts=0, apply_ts=0, pushed=None)
        self.lay = lay
        assert lay.total() <= fabric.heap_bytes, "heap too small"
        dev = fabric.device
        self.sync = torch.zeros(4 * max(1, len(layers)), dtype=torch.int32, device=dev)   # per layer: push, apply arrivals
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    @staticmethod
    def heap_bytes(layers: Dict[int, int], world: int, partition_thr: int = 1000, ring: int = 2) -> int:
        total = 0
        for lid, n in layers.items():
            mx = _up4(n) if n < partition_thr else _up4((n + world - 1) // world) + 8
            total += (mx * 4 + 256) * (ring * world + 1) + 4 * (ring * world + 2) + 512
        return total + 4096

    def segments(self, lid: int, n: int) -> List[int]:
        """Element boundaries of the shards for layer ``lid`` (multiples of four elements, so that every
        slice starts on a 16-byte boundary)."""
        S = self.S
        if n < self.thr:
            owner = (lid * 991) % S
            return [0 if s <= owner else n for s in range(S + 1)]
        return [(n * s // S) // 4 * 4 for s in range(S)] + [n]

    def _p(self, rank, off):
        return self.fabric.ptr(rank, off)

    def _inbox(self, m, owner: int, q: int, src: int) -> int:
        return self._p(owner, m["inbox"] + ((q * self.S + src) * m["cap"]) * 4)

    def _ready(self, m, owner: int, q: int, src: int) -> int:
        return self._p(owner, m["flags"] + 4 * (1 + q * self.S + src))

    def push(self, lid: int, data: torch.Tensor, wait_iters: int = 0, stream=None) -> int:
        """Worker side of the layer's next round: returns its timestamp."""
        m = self.meta[lid]
        assert data.numel() == m["n"] and data.dtype == torch.float32 and data.is_contiguous()
        ts = m["push_ts"]
        m["push_ts"] += 1
        q = ts % self.ring
        a = _Push()
        a.S, a.ts1, a.data = self.S, ts + 1, ptr(data)
        a.need_applied, a.wait_iters = max(0, ts + 1 - self.ring), wait_iters
        for s in range(self.S + 1):
            a.seg_begin[s] = m["seg"][s]
        for s in range(self.S):
            a.inbox[s] = self._inbox(m, s, q, self.rank)
            a.ready[s] = self._ready(m, s, q, self.rank)
            a.applied[s] = self._p(s, m["flags"])
        a.done, a.status = self.sync.data_ptr() + 16 * m["idx"], ptr(self.status)
        check(self.L.psb_layer_push(C.byref(a), stream_ptr(stream)), "layer_push")
        ev = m["pushed"] = m["pushed"] or torch.cuda.Event()
        ev.record(stream if stream is not None else torch.cuda.current_stream())
        return ts

    def apply(self, lid: int, alive=None, wait_iters: int = 0, stream=None):
        """Owner side of the layer's next unapplied round (every rank calls it once per round)."""
        m = self.meta[lid]
        ts = m["apply_ts"]
        m["apply_ts"] += 1
        q = ts % self.ring
        n = m["seg"][self.rank + 1] - m["seg"][self.rank]
        st = stream if stream is not None else torch.cuda.current_stream()
        if m["pushed"] is not None:
            st.wait_event(m["pushed"])          # this rank's own push: ordered by the stream, not by a device wait
        a = _Apply()
        a.S, a.ts1, a.updater, a.lr, a.n = self.S, ts + 1, self.updater, self.lr, n
        a.data = self._p(self.rank, m["data"])
        for r in range(self.S):
            a.inbox[r] = self._inbox(m, self.rank, q, r)
            a.ready[r] = self._ready(m, self.rank, q, r)
            a.alive[r] = 1 if (alive is None or alive[r]) else 0
        a.wait_iters = wait_iters
        a.applied, a.done, a.status = self._p(self.rank, m["flags"]), self.sync.data_ptr() + 16 * m["idx"] + 8, ptr(self.status)
        check(self.L.psb_layer_apply(C.byref(a), stream_ptr(stream)), "layer_apply")

    def pull(self, lid: int, out: torch.Tensor, wait_for_round: int = 0, wait_iters: int = 0, stream=None):
        """Gather the layer from its owners into ``out``; waits until the owners
        have applied ``wait_for_round`` pushes."""
        m = self.meta[lid]
        assert out.numel() == m["n"] and out.dtype == torch.float32 and out.is_contiguous()
        a = _Pull()
        a.S, a.need_applied, a.out = self.S, wait_for_round, ptr(out)
        a.wait_iters = wait_iters
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
        _lib.check_status(self.status, what, reset=(self.sync,))


def fabric_copy(src_ptr: int, dst_ptr: int, nbytes: int, mode: int = 0, sink=None, stream=None):
    """16-byte copy kernel between two device addresses, either of which may be a peer's memory
    (mode 0: copy; mode 1: read-only pass over ``src``)."""
    L = _declare()
    check(L.psb_fabric_copy(src_ptr, dst_ptr, nbytes, mode, ptr(sink), stream_ptr(stream)), "fabric_copy")
