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

Values may be ``k`` floats wide (``KVVector<K,V>(buffer_value, k)``,
``parameter/kv_vector.h:43-104``): pushes take and pulls return ``(n, k)`` arrays.
``channels`` independent key/value sets share the object (``kv[chl]`` in the
reference): ``push`` / ``pull`` take a ``channel``. With ``buffer_value=True`` a
push round is not merged into the channel: the owner finds what every worker
sent under :meth:`buffer` (per source, keys and values), and merges it itself
(:meth:`apply_buffer`, or by pushing something else), which is the reference's
aggregation idiom (``kv_vector.h:182-207``, ``test/kv_vector_buffer_ps.cc:10-59``).

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
    def __init__(self, plane: DataPlane, max_keys: int = 1 << 20, buffer_value: bool = False):
        self.plane = plane
        self.max_keys = max_keys
        self.k = plane.width
        self.buffer_value = buffer_value
        self._push_round_of: Dict[int, int] = {}      # timestamp -> push round (for buffer())
        self.dev = plane.device
        self._time = -1
        self._round = 0                       # push rounds seen by the owners
        self._pull_round = 0                  # exchange rounds (pulls)
        self._events: Dict[int, torch.cuda.Event] = {}
        self._callbacks: Dict[int, Callable] = {}
        self._results: Dict[int, torch.Tensor] = {}
        self._bufs: List[LocalBatch] = [LocalBatch(1, max_keys, plane.S, self.dev) for _ in range(4)]
        if self.k > 1:
            for b in self._bufs:                      # k values per key, key-major
                b.grad = torch.zeros(max_keys * self.k, dtype=torch.float32, device=self.dev)
        self._next_buf = 0
        self.stream = torch.cuda.Stream(device=self.dev)

    @classmethod
    def create(cls, fabric_or_none=None, *, table_capacity: int = 1 << 20, max_keys: int = 1 << 18,
               opt: Optional[OptimizerConfig] = None, ring: int = 4, quant: str = "none", world: int = 1,
               exchange: bool = True, key_cache: bool = False, k: int = 1, channels: int = 1,
               buffer_value: bool = False):
        """``fabric_or_none``: an existing fabric whose heap is large enough, or None to
        make one: over the default process group when ``torch.distributed`` is
        initialised with more than one rank, else a single-GPU heap. ``key_cache``
        turns the key-caching filter on: a pull whose key list equals the previous
        pull's sends no keys (decided inside the exchange kernel)."""
        pc = PlaneConfig(table_capacity=table_capacity, inbox_cap=max_keys, ring=ring, quant=quant,
                         pull_cap=max_keys if exchange else 0, key_cache=key_cache, width=k, channels=channels)
        fab = fabric_or_none
        if fab is None:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                fab = Fabric.from_process_group(heap_layout(pc, dist.get_world_size()).total())
            else:
                fab = Fabric.single(heap_layout(pc, world).total())
        return cls(DataPlane(fab, pc, opt or OptimizerConfig(algo="sum")), max_keys, buffer_value=buffer_value)

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
        # A request with the very key tensor of the request before it (the usual push-then-pull pair; same
        # object, not written to since) reuses that request's key buffer and owner offsets: three launches less.
        tag = (id(keys), keys._version, keys.data_ptr(), keys.numel())
        if tag == self.__dict__.get("_last_keys_tag"):
            return self._last_buf
        b = self._bufs[self._next_buf]
        self._next_buf = (self._next_buf + 1) % len(self._bufs)
        b.set_keys(keys, self.plane.bounds)
        self._last_keys_tag, self._last_buf, self._last_keys = tag, b, keys      # (keeps the tensor, and so its id, alive)
        return b

    @staticmethod
    def _as_keys(keys, dev) -> torch.Tensor:
        if isinstance(keys, torch.Tensor):
            return keys.to(dev)
        k = np.ascontiguousarray(np.asarray(keys, dtype=np.uint64))
        assert (np.diff(k.astype(np.float64)) > 0).all() if len(k) > 1 else True, "keys must be sorted and unique"
        return torch.from_numpy(k.view(np.int64)).to(dev)

    def push(self, keys, values, ts: Optional[int] = None, wait: Optional[List[int]] = None, callback=None,
             channel: int = 0) -> int:
        """Push sorted unique uint64 keys with one value (``k`` values: an ``(n, k)`` array) each into
        ``channel``; returns the timestamp. Both halves of the round are enqueued here: the worker half
        (values into the owners' inboxes) and this rank's owner half (merge of the round)."""
        ts = self._stamp(ts)
        self._begin(wait)
        rnd = self.push_only(keys, values)
        self._push_round_of[ts] = rnd
        self.apply_round(rnd, channel=channel)
        self._finish(ts, callback)
        return ts

    def push_only(self, keys, values) -> int:
        """The worker half of a push round: the values go into the owners' inboxes. Returns the round.
        The owner half is :meth:`apply_round`; :meth:`push` does both, the node-level customers
        (``parameter/kv_nodes.py``) let the server node decide when the round is merged."""
        k = self._as_keys(keys, self.dev)
        with torch.cuda.stream(self.stream):
            b = self._buffer(k)
            n = k.numel()
            if n:
                v = torch.as_tensor(values, dtype=torch.float32).to(self.dev).flatten()
                assert v.numel() == n * self.k, f"{n} keys of width {self.k} need {n * self.k} values"
                b.grad[:n * self.k].copy_(v)
            rnd = self._round
            self._round += 1
            self.plane.push(b, rnd, with_gradient=False, stream=self.stream)
        return rnd

    def apply_round(self, rnd: int, channel: int = 0):
        """The owner half of push round ``rnd``: merge what every live worker sent (a buffered container
        only consumes the round: its ring slot becomes reusable later, the values stay unmerged)."""
        with torch.cuda.stream(self.stream):
            self.plane.apply(rnd, channel=channel, stream=self.stream,
                             opt=OptimizerConfig(algo="keep") if self.buffer_value else None)

    def buffer(self, ts: int):
        """What this rank, as an owner, received in the push with timestamp ``ts``: one
        ``(keys uint64 array, values tensor (n, k))`` pair per source rank. Readable until ``ring - 1``
        further rounds have been pushed (the inbox slot is then reused)."""
        self.wait(ts) if ts in self._events else None
        rnd = self._push_round_of[ts]
        p = self.plane
        q = rnd % p.cfg.ring
        torch.cuda.current_stream(self.dev).synchronize()
        out = []
        for r in range(p.S):
            word = 8 + p.cfg.ring * p.S + q * p.S + r
            n = int(p.ctrl[word].item())
            ko = p.layout["inbox_keys"] + ((q * p.S + r) * p.cfg.inbox_cap) * 8
            vo = p.layout["inbox_vals"] + ((q * p.S + r) * p.cfg.inbox_cap) * 4 * self.k
            keys = p.fabric.view(ko, (n,), torch.int64).cpu().numpy().view(np.uint64)
            vals = p.fabric.view(vo, (n * self.k,), torch.float32).clone().view(n, self.k)
            out.append((keys, vals))
        return out

    def apply_buffer(self, ts: int, channel: int = 0):
        """Merge the buffered round ``ts`` into ``channel`` (sum over the workers, added to the stored values)."""
        rnd = self._push_round_of[ts]
        with torch.cuda.stream(self.stream):
            self.plane.apply(rnd, channel=channel, stream=self.stream, opt=OptimizerConfig(algo="sum"))

    def pull(self, keys, ts: Optional[int] = None, wait: Optional[List[int]] = None, callback=None,
             channel: int = 0) -> int:
        """Pull the values of ``keys`` from ``channel``; the result is available from :meth:`result` after :meth:`wait`."""
        ts = self._stamp(ts)
        k = self._as_keys(keys, self.dev)
        self._begin(wait)
        with torch.cuda.stream(self.stream):
            b = self._buffer(k)
            # the owners must have applied every round pushed so far
            if self.plane.cfg.pull_cap:
                rnd = self._pull_round
                self._pull_round += 1
                self.plane.pull_exchange(b, rnd, need_applied=self._round, with_margins=False, channel=channel,
                                         stream=self.stream)
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

    def discard(self, ts: int):
        """Forget request ``ts`` (its event, callback and pulled values) without waiting for it."""
        self._events.pop(ts, None)
        self._callbacks.pop(ts, None)
        self._results.pop(ts, None)

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
