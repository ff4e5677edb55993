"""Push/Pull containers on the device data plane with the reference's calling
conventions: timestamps, ``wait`` dependencies, callbacks and ``wait(ts)``.

:class:`DeviceKVMap` is the device form of ``KVMap`` (``parameter/kv_map.h:32-66``):
the server side keeps a hash table and runs an entry update (FTRL / AdaGrad / SGD
/ plain sum) on every pushed key; :class:`DeviceKVVector` is the ``sum`` flavour
used like ``KVVector`` with ``PLUS`` merging (``parameter/kv_vector.h:171-211``).
Every rank calls ``push`` for every round (possibly with no keys), because the
owner aggregates one round from all live workers -- the device counterpart of
"an empty but valid slice is still sent" (``system/message.h:136-137``).

With ``exchange=True`` (the default) pulls use the two-sided exchange kernel (keys
to the owners in bulk, weights back in bulk), which is what NVLink likes; then
``pull`` is collective as well: every rank calls it for every round, possibly
with no keys. ``exchange=False`` keeps the one-sided pull (remote probes), which
any rank may call on its own.

Timestamps are per object and increase by one per request unless given.
Requests run in stream order; ``wait=[t]`` makes a request's kernels wait for
the CUDA event of request ``t``, and ``wait(ts)`` blocks the host until request
``ts`` has finished on the device (then runs its callback).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from ..ops.localize import LocalBatch
from ..parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig, heap_layout
from ..parallel.fabric import Fabric


class DeviceKVMap:
    def __init__(self, plane: DataPlane, max_keys: int = 1 << 20):
        self.plane = plane
        self.max_keys = max_keys
        self.dev = plane.device
        self._time = -1
        self._round = 0                       # push rounds seen by the owners
        self._pull_round = 0                  # exchange rounds (pulls)
        self._events: Dict[int, torch.cuda.Event] = {}
        self._callbacks: Dict[int, Callable] = {}
        self._results: Dict[int, torch.Tensor] = {}
        self._bufs: List[LocalBatch] = [LocalBatch(1, max_keys, plane.S, self.dev) for _ in range(4)]
        self._next_buf = 0
        self.stream = torch.cuda.Stream(device=self.dev)

    @classmethod
    def create(cls, fabric_or_none=None, *, table_capacity: int = 1 << 20, max_keys: int = 1 << 18,
               opt: Optional[OptimizerConfig] = None, ring: int = 4, quant: str = "none", world: int = 1,
               exchange: bool = True):
        """``fabric_or_none``: an existing fabric whose heap is large enough, or None to
        make one: over the default process group when ``torch.distributed`` is
        initialised with more than one rank, else a single-GPU heap."""
        pc = PlaneConfig(table_capacity=table_capacity, inbox_cap=max_keys, ring=ring, quant=quant,
                         pull_cap=max_keys if exchange else 0)
        fab = fabric_or_none
        if fab is None:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                fab = Fabric.from_process_group(heap_layout(pc, dist.get_world_size()).total())
            else:
                fab = Fabric.single(heap_layout(pc, world).total())
        return cls(DataPlane(fab, pc, opt or OptimizerConfig(algo="sum")), max_keys)

    def _stamp(self, ts: Optional[int]) -> int:
        ts = self._time + 1 if ts is None or ts < 0 else ts
        self._time = max(self._time, ts)
        return ts

    def _begin(self, wait: Optional[List[int]]):
        self.stream.wait_stream(torch.cuda.current_stream(self.dev))
        for t in wait or []:
            ev = self._events.get(t)
            if ev is not None:
                self.stream.wait_event(ev)

    def _finish(self, ts: int, callback):
        ev = torch.cuda.Event()
        ev.record(self.stream)
        self._events[ts] = ev
        if callback is not None:
            self._callbacks[ts] = callback

    def _buffer(self, keys: torch.Tensor) -> LocalBatch:
        b = self._bufs[self._next_buf]
        self._next_buf = (self._next_buf + 1) % len(self._bufs)
        b.set_keys(keys, self.plane.bounds)
        return b

    @staticmethod
    def _as_keys(keys, dev) -> torch.Tensor:
        if isinstance(keys, torch.Tensor):
            return keys.to(dev)
        k = np.ascontiguousarray(np.asarray(keys, dtype=np.uint64))
        assert (np.diff(k.astype(np.float64)) > 0).all() if len(k) > 1 else True, "keys must be sorted and unique"
        return torch.from_numpy(k.view(np.int64)).to(dev)

    def push(self, keys, values, ts: Optional[int] = None, wait: Optional[List[int]] = None, callback=None) -> int:
        """Push (sorted unique uint64 keys, float values); returns the timestamp."""
        ts = self._stamp(ts)
        k = self._as_keys(keys, self.dev)
        self._begin(wait)
        with torch.cuda.stream(self.stream):
            b = self._buffer(k)
            n = k.numel()
            if n:
                b.grad[:n].copy_(torch.as_tensor(values, dtype=torch.float32).to(self.dev).flatten())
            rnd = self._round
            self._round += 1
            self.plane.push(b, rnd, with_gradient=False, stream=self.stream)
            self.plane.apply(rnd, stream=self.stream)
        self._finish(ts, callback)
        return ts

    def pull(self, keys, ts: Optional[int] = None, wait: Optional[List[int]] = None, callback=None) -> int:
        """Pull the weights of ``keys``; the result is available from :meth:`result` after :meth:`wait`."""
        ts = self._stamp(ts)
        k = self._as_keys(keys, self.dev)
        self._begin(wait)
        with torch.cuda.stream(self.stream):
            b = self._buffer(k)
            # the owners must have applied every round pushed so far
            if self.plane.cfg.pull_cap:
                rnd = self._pull_round
                self._pull_round += 1
                self.plane.pull_exchange(b, rnd, need_applied=self._round, with_margins=False, stream=self.stream)
                self._results[ts] = self.plane.response_weights(rnd, k.numel()).clone()
            else:
                self.plane.pull_margin(b, need_applied=self._round, with_margins=False, stream=self.stream)
                self._results[ts] = b.w_local[:k.numel()].clone()
        self._finish(ts, callback)
        return ts

    def wait(self, ts: int):
        ev = self._events.pop(ts, None)
        if ev is not None:
            ev.synchronize()
        self.plane.check_status("kv")
        cb = self._callbacks.pop(ts, None)
        if cb is not None:
            cb()

    def result(self, ts: int) -> torch.Tensor:
        return self._results.pop(ts)

    def write_to_file(self, path: str):
        """``key<TAB>value`` per non-zero entry of this shard."""
        from ..app.linear import write_model
        keys, w = self.plane.dump_nonzero()
        write_model(path, keys.numpy(), w.numpy())


class DeviceKVVector(DeviceKVMap):
    """``sum`` entries: a push adds into the stored values (KVVector PLUS semantics)."""

    @classmethod
    def create(cls, fabric_or_none=None, **kw):
        kw.setdefault("opt", OptimizerConfig(algo="sum"))
        return super().create(fabric_or_none, **kw)
