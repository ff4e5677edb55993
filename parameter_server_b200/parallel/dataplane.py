"""Device data plane: one server shard plus one worker endpoint per GPU.

The heap of every rank holds, at identical offsets,

* ``ctrl``   -- flag words: ``applied`` (timestamp+1 of the last applied push
  round), and per (ring slot, source) a ``ready`` flag and a record ``count``;
* ``table``  -- the shard's open-addressing table (32-byte entries: key, w,
  optimiser state, per-round gradient accumulator, epoch tag);
* ``inbox``  -- per (ring slot, source) a key array and a value array that the
  source's push kernel fills with peer stores.

A push of timestamp ``t`` uses ring slot ``t % ring``; a worker may reuse a slot
once the owner has applied round ``t - ring``. A pull at step ``t`` with bounded
delay ``tau`` waits until every owner has applied round ``t - tau - 1``. Both are
waits on the owners' ``applied`` counters, i.e. the device form of the
reference's per-sender timestamp trackers and ``wait_time`` dependencies
(``system/remote_node.h:13-32``, ``system/executor.cc:169-230``).

Push rounds are aggregated per timestamp at the owner: gradients of the same key
from different workers are summed and the optimiser runs once on the sum (the
buffered-aggregation semantics of ``parameter/kv_vector.h:182-207``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..ops import _lib
from ..ops._lib import (ApplyParams, Optimizer, PullParams, PushParams, check, ptr, stream_ptr)
from ..utils.range import Range, shard_bounds
from .fabric import Fabric, HeapLayout

CTRL_WORDS = 1024


@dataclass
class OptimizerConfig:
    algo: str = "ftrl"            # ftrl | adagrad | sgd | sum | keep (consume a round, leave the values)
    alpha: float = 0.1
    beta: float = 1.0
    l1: float = 1.0
    l2: float = 0.1
    lr_type: str = "decay"        # decay: alpha/(x+beta) ; constant: alpha

    def to_c(self) -> Optimizer:
        algo = {"ftrl": _lib.ALGO_FTRL, "adagrad": _lib.ALGO_ADAGRAD, "sgd": _lib.ALGO_SGD,
                "sum": _lib.ALGO_SUM, "keep": _lib.ALGO_KEEP}[self.algo]
        lr = _lib.LR_CONSTANT if self.lr_type == "constant" else _lib.LR_DECAY
        return Optimizer(algo, lr, self.alpha, self.beta, self.l1, self.l2)


@dataclass
class PlaneConfig:
    table_capacity: int                     # slots per shard, power of two
    inbox_cap: int                          # records per (owner, source) inbox
    ring: int = 2                           # inbox ring slots (bounded delay tau => tau+2)
    key_range: Range = field(default_factory=Range.all)
    quant: str = "none"                     # none | int8 | fp16 (fixed-point filter on pushes)
    ordered_slots: bool = False             # keys are uniformly hashed: order-preserving slot map
    key_cache: bool = False                 # key-caching filter: skip keys (push) and probes (pull) on a repeated key list
    pull_cap: int = 0                       # unique keys per worker minibatch for the two-sided pull (0: off)
    width: int = 1                          # values per key (k of KVVector<K,V>(.., k)); k > 1: sum entries, exchange pull
    channels: int = 1                       # independent key/value sets (the KVVector channels), one table each

    def quant_code(self) -> int:
        return {"none": _lib.QUANT_NONE, "int8": _lib.QUANT_INT8, "fp16": _lib.QUANT_FP16}[self.quant]


def heap_layout(cfg: PlaneConfig, world: int) -> HeapLayout:
    assert cfg.table_capacity & (cfg.table_capacity - 1) == 0, "table capacity must be a power of two"
    assert cfg.table_capacity < (1 << 31)
    assert 8 + 3 * cfg.ring * world <= CTRL_WORDS
    lay = HeapLayout()
    k = max(1, cfg.width)
    lay.add("ctrl", CTRL_WORDS * 4)
    lay.add("table", cfg.channels * cfg.table_capacity * 32)
    if k > 1:
        lay.add("wide_vals", cfg.channels * cfg.table_capacity * k * 4)
    lay.add("inbox_keys", cfg.ring * world * cfg.inbox_cap * 8)
    lay.add("inbox_vals", cfg.ring * world * cfg.inbox_cap * k * 4 + 256)
    if cfg.pull_cap:
        # two-sided pull: request areas per (parity, source), response buffer per parity, flags
        lay.add("xflags", 4 * (16 * world + 16))
        lay.add("req_keys", 2 * world * cfg.inbox_cap * 8)
        lay.add("resp_w", 2 * cfg.pull_cap * k * 4)
    return lay


class DataPlane:
    """Server shard + worker endpoint of one rank."""

    def __init__(self, fabric: Fabric, cfg: PlaneConfig, opt: OptimizerConfig):
        self.fabric, self.cfg, self.opt = fabric, cfg, opt
        self.rank, self.S = fabric.rank, fabric.world
        assert self.S <= _lib.MAX_SHARDS
        self.layout = heap_layout(cfg, self.S)
        assert self.layout.total() <= fabric.heap_bytes, "heap too small for this configuration"
        dev = fabric.device
        self.device = dev
        self.bounds_host = shard_bounds(cfg.key_range, self.S)
        self.bounds = torch.tensor([b if b < (1 << 63) else b - (1 << 64) for b in self.bounds_host],
                                   dtype=torch.int64, device=dev)
        # local scratch (zero-initialised); one word group per kernel kind
        self.sync_words = torch.zeros(64, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        # Slots found per (source, record). The exchange pull of round t fills them and the
        # apply of round t consumes them up to tau rounds later, while the pulls of the next
        # rounds already run: one copy per ring slot, like the inboxes. Without the exchange
        # pull only copy 0 is used (scratch of apply, and the key-caching filter's memory).
        n_sc = cfg.ring if cfg.pull_cap else 1
        self.slot_cache = torch.zeros((n_sc, self.S, cfg.inbox_cap), dtype=torch.int32, device=dev)
        # For the merge of several sources in apply: the exchange pull notes where each of `tiles` equal
        # parts of this shard's key range starts in every source's list (about 400 records per part
        # when the lists are full), one set of notes per ring slot like the slots.
        self.tiles = 0
        self.tile_off = None
        if cfg.pull_cap and self.S > 1 and max(1, cfg.width) == 1:
            self.tiles = min(1 << 16, max(64, 1 << max(0, (cfg.inbox_cap // 400)).bit_length()))
            self.tile_off = torch.zeros((n_sc, self.S, self.tiles + 1), dtype=torch.int32, device=dev)
        self.push_stats = torch.zeros(4, dtype=torch.float64, device=dev)   # d_nnz, w2, dw2, n
        self.pull_stats = torch.zeros(4, dtype=torch.float64, device=dev)   # loss, correct, rows
        self.alive = [True] * self.S
        # key-caching filter state: signature of the previous key list, and the slots found for it
        self.sig_state = torch.zeros(4, dtype=torch.int32, device=dev)
        self.sig_scratch = torch.zeros(4, dtype=torch.int32, device=dev)
        self.kc_state = torch.zeros(4, dtype=torch.int64, device=dev)       # exchange pull: fingerprints by round parity
        self.pull_slot_cache = None
        # order-preserving slot multiplier per shard: floor(capacity * 2^64 / range_size)
        self.slot_mult = []
        for s in range(self.S):
            size = self.bounds_host[s + 1] - self.bounds_host[s]
            m = (cfg.table_capacity << 64) // size if (cfg.ordered_slots and size > cfg.table_capacity) else 0
            self.slot_mult.append(m if m < (1 << 64) else 0)
        self.applied_ts1 = 0
        self.ctrl = fabric.view(self.layout["ctrl"], (CTRL_WORDS,), torch.int32)
        self.width = max(1, cfg.width)
        assert self.width == 1 or (cfg.pull_cap and opt.algo in ("sum", "keep")), \
            "values of width k > 1 are sum entries (KVVector) and use the exchange pull"
        check(_lib.lib().psb_table_init(fabric.ptr(self.rank, self.layout["table"]),
                                        cfg.channels * cfg.table_capacity, stream_ptr()), "table init")
        if self.width > 1:
            fabric.view(self.layout["wide_vals"], (cfg.channels * cfg.table_capacity * self.width,), torch.float32).zero_()

    # ---------------------------------------------------------------- addresses
    def _slot_cache_ptr(self, ts: int, source: int) -> int:
        q = ts % self.slot_cache.shape[0]
        return self.slot_cache.data_ptr() + (q * self.S + source) * self.cfg.inbox_cap * 4

    def _ctrl(self, rank: int, word: int) -> int:
        return self.fabric.ptr(rank, self.layout["ctrl"] + 4 * word)

    def _ready(self, owner: int, q: int, src: int) -> int:
        return self._ctrl(owner, 8 + q * self.S + src)

    def _count(self, owner: int, q: int, src: int) -> int:
        return self._ctrl(owner, 8 + self.cfg.ring * self.S + q * self.S + src)

    def _mode(self, owner: int, q: int, src: int) -> int:
        return self._ctrl(owner, 8 + 2 * self.cfg.ring * self.S + q * self.S + src)

    def _inbox_keys(self, owner: int, q: int, src: int) -> int:
        return self.fabric.ptr(owner, self.layout["inbox_keys"] + ((q * self.S + src) * self.cfg.inbox_cap) * 8)

    def _inbox_vals(self, owner: int, q: int, src: int) -> int:
        return self.fabric.ptr(owner, self.layout["inbox_vals"] + ((q * self.S + src) * self.cfg.inbox_cap) * 4 * self.width)

    def _bar(self, kind: int) -> int:
        return self.sync_words.data_ptr() + 16 * kind

    def _done(self, kind: int) -> int:
        return self.sync_words.data_ptr() + 16 * kind + 8

    def table_ptr(self, rank: Optional[int] = None, channel: int = 0) -> int:
        assert 0 <= channel < self.cfg.channels
        return self.fabric.ptr(self.rank if rank is None else rank,
                               self.layout["table"] + channel * self.cfg.table_capacity * 32)

    def wide_vals_ptr(self, channel: int = 0) -> int:
        if self.width == 1:
            return 0
        return self.fabric.ptr(self.rank, self.layout["wide_vals"] + channel * self.cfg.table_capacity * self.width * 4)

    # ---------------------------------------------------------------- key-caching filter
    def key_signature(self, b, stream=None):
        """Signature of ``b``'s key list (crc32c of its head + a fingerprint of
        the whole list) compared on the device with the previous list's; leaves
        the hit flag in ``b.key_hit``. Call once per minibatch, before the pull."""
        check(_lib.lib().psb_key_signature(ptr(b.ukeys), ptr(b.n_unique), b.max_nnz, ptr(self.sig_scratch),
                                           ptr(self.sig_state), ptr(b.key_hit), ptr(b.key_sig), stream_ptr(stream)),
              "key_signature")
        if self.pull_slot_cache is None or self.pull_slot_cache.numel() < b.max_nnz:
            self.pull_slot_cache = torch.full((b.max_nnz,), -1, dtype=torch.int32, device=self.device)

    # ---------------------------------------------------------------- worker: pull (+ margins)
    def pull_margin(self, b, *, need_applied: int = 0, with_margins: bool = True, loss: int = 0,
                    insert: bool = False, auc_hist: Optional[torch.Tensor] = None, stream=None):
        """F2 on a localised batch ``b`` (see :class:`~parameter_server_b200.ops.localize.LocalBatch`)."""
        p = PullParams()
        p.S, p.insert = self.S, int(insert)
        for s in range(self.S):
            p.table[s] = self.table_ptr(s)
            p.mask[s] = self.cfg.table_capacity - 1
            p.key_begin[s] = self.bounds_host[s]
            p.slot_mult[s] = self.slot_mult[s]
            p.applied[s] = self._ctrl(s, 0)
        p.need_applied = need_applied
        p.ukeys, p.n_unique, p.own_off = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off)
        p.w_local, p.slot_local, p.grad_zero = ptr(b.w_local), ptr(b.slot_local), ptr(b.grad)
        if self.cfg.key_cache and self.pull_slot_cache is not None:
            p.slot_local, p.key_hit = ptr(self.pull_slot_cache), ptr(b.key_hit)
        if with_margins:
            p.row_ptr, p.n_rows, p.fixed_z = ptr(b.row_ptr), b.n_rows, b.fixed_z
            p.csr_col, p.csr_val, p.y = ptr(b.csr_col), ptr(b.csr_val), ptr(b.y)
            p.gcoef, p.margin = ptr(b.gcoef), ptr(b.margin)
        else:
            p.n_rows = 0
        p.loss = loss
        p.stats, p.auc_hist = ptr(self.pull_stats), ptr(auc_hist)
        p.bar, p.status = self._bar(0), ptr(self.status)
        check(_lib.lib().psb_pull_margin(C.byref(p), stream_ptr(stream)), "pull_margin")

    # ---------------------------------------------------------------- two-sided pull (+ margins)
    def _xflag(self, rank: int, kind: int, par: int, idx: int) -> int:
        """kind 0: req_ready, 1: resp_ready, 2/3: the two request header words."""
        return self.fabric.ptr(rank, self.layout["xflags"] + 4 * (((kind * 2) + par) * self.S + idx))

    def pull_exchange(self, b, ts: int, *, need_applied: int = 0, with_margins: bool = True, loss: int = 0,
                      auc_hist: Optional[torch.Tensor] = None, phases: int = 7, wait_iters: int = 0, channel: int = 0,
                      stream=None):
        """Exchange form of F2 for round ``ts``: keys go to the owners in bulk, the
        owners look them up (inserting absent keys), remember the slots for the push
        of the same round and store the weights into this worker's response buffer.
        After it, ``push(..., send_keys=False)`` + ``apply`` reuse those slots."""
        from ..ops._lib import PullExchangeParams
        cfg = self.cfg
        assert cfg.pull_cap >= b.max_nnz, "pull_cap must cover the largest minibatch's unique keys"
        par = ts & 1

        def build():
            p = PullExchangeParams()
            p.S, p.me, p.req_cap = self.S, self.rank, cfg.inbox_cap
            req_bytes = cfg.inbox_cap * 8
            for s in range(self.S):
                p.req_keys[s] = self.fabric.ptr(s, self.layout["req_keys"] + (par * self.S + self.rank) * req_bytes)
                p.req_ready[s] = self._xflag(s, 0, par, self.rank)
                p.my_req_keys[s] = self.fabric.ptr(self.rank, self.layout["req_keys"] + (par * self.S + s) * req_bytes)
                p.my_req_ready[s] = self._xflag(self.rank, 0, par, s)
                p.resp_w[s] = self.fabric.ptr(s, self.layout["resp_w"] + par * cfg.pull_cap * 4 * self.width)
                p.resp_ready[s] = self._xflag(s, 1, par, self.rank)
                p.my_resp_ready[s] = self._xflag(self.rank, 1, par, s)
                p.slot_cache[s] = self._slot_cache_ptr(ts, s)
                p.alive[s] = 1 if self.alive[s] else 0
                # header = two consecutive words {count, base} per (parity, source)
                p.req_hdr[s] = self.fabric.ptr(s, self.layout["xflags"] + 4 * (8 * self.S + (par * self.S + self.rank) * 2))
                p.my_req_hdr[s] = self.fabric.ptr(self.rank, self.layout["xflags"] + 4 * (8 * self.S + (par * self.S + s) * 2))
                p.slot_cache_prev[s] = self._slot_cache_ptr(ts - 1, s) if ts > 0 else self._slot_cache_ptr(ts, s)
            p.table, p.mask = self.table_ptr(channel=channel), cfg.table_capacity - 1
            p.key_begin, p.slot_mult = self.bounds_host[self.rank], self.slot_mult[self.rank]
            p.applied = self._ctrl(self.rank, 0)
            p.width, p.wide_vals = self.width, self.wide_vals_ptr(channel)
            p.my_resp_w = self.fabric.ptr(self.rank, self.layout["resp_w"] + par * cfg.pull_cap * 4 * self.width)
            p.stats = ptr(self.pull_stats)
            p.done, p.status = self.sync_words.data_ptr() + 48, ptr(self.status)
            if self.tile_off is not None:
                n_sc = self.tile_off.shape[0]
                p.tile_off = self.tile_off[ts % n_sc].data_ptr()
                p.tile_off_prev = self.tile_off[(ts - 1) % n_sc].data_ptr()
                p.tiles = self.tiles
                p.key_end = self.bounds_host[self.rank + 1] & ((1 << 64) - 1)      # 2^64 is passed as 0
            return p
        # everything that depends on the round only through its ring slot and parity is filled once
        p = self._params("pull_exchange", (ts % (2 * cfg.ring) if ts > 0 else -1, channel), build)
        p.ts1, p.need_applied, p.wait_iters, p.phases = ts + 1, need_applied, wait_iters, phases
        assert self.width == 1 or not with_margins, "margins need scalar values"
        p.ukeys, p.n_unique, p.own_off, p.grad_zero = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off), ptr(b.grad)
        if with_margins:
            p.row_ptr, p.n_rows, p.fixed_z = ptr(b.row_ptr), b.n_rows, b.fixed_z
            p.csr_col, p.csr_val, p.y = ptr(b.csr_col), ptr(b.csr_val), ptr(b.y)
            p.gcoef, p.margin = ptr(b.gcoef), ptr(b.margin)
        p.loss, p.auc_hist = loss, ptr(auc_hist)
        if cfg.key_cache and phases == 7:
            # the key-caching filter is decided inside the kernel (needs all three roles in one launch:
            # the fingerprint pass ends with a grid barrier)
            p.key_cache, p.kc_state, p.bar = 1, ptr(self.kc_state), self.sync_words.data_ptr() + 64
        check(_lib.lib().psb_pull_exchange(C.byref(p), stream_ptr(stream)), "pull_exchange")

    def response_weights(self, ts: int, n: int) -> torch.Tensor:
        """The weights this worker received in the exchange of round ``ts``."""
        k = self.width
        v = self.fabric.view(self.layout["resp_w"] + (ts & 1) * self.cfg.pull_cap * 4 * k, (n * k,), torch.float32)
        return v if k == 1 else v.view(n, k)

    # ---------------------------------------------------------------- worker: push
    def push(self, b, ts: int, *, with_gradient: bool = True, send_keys: bool = True, stream=None):
        """F1a: push round ``ts`` of batch ``b``. With ``with_gradient`` the values
        are X^T gcoef computed in the kernel; otherwise ``b.grad`` is sent as is."""
        cfg = self.cfg
        q = ts % cfg.ring

        def build():
            p = PushParams()
            p.S, p.inbox_cap, p.quant, p.width = self.S, cfg.inbox_cap, cfg.quant_code(), self.width
            for s in range(self.S):
                p.inbox_keys[s] = self._inbox_keys(s, q, self.rank)
                p.inbox_vals[s] = self._inbox_vals(s, q, self.rank)
                p.ready[s] = self._ready(s, q, self.rank)
                p.count[s] = self._count(s, q, self.rank)
                p.mode[s] = self._mode(s, q, self.rank)
                p.applied[s] = self._ctrl(s, 0)
            p.bar, p.done, p.status = self._bar(1), self._done(1), ptr(self.status)
            return p
        p = self._params("push", q, build)
        p.ts1, p.send_keys = ts + 1, int(send_keys)
        if cfg.key_cache:
            p.key_hit = ptr(b.key_hit)
        p.need_applied = max(0, ts + 1 - cfg.ring)
        p.ukeys, p.n_unique, p.own_off = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off)
        if with_gradient:
            p.nnz = b.nnz
            p.csc_row, p.csc_val = ptr(b.csc_row), ptr(b.csc_val)
            p.flagbits, p.wordbase, p.gcoef = ptr(b.flagbits), ptr(b.wordbase), ptr(b.gcoef)
        else:
            p.nnz = 0
        p.grad = ptr(b.grad)
        assert self.width == 1 or not with_gradient
        check(_lib.lib().psb_push(C.byref(p), stream_ptr(stream)), "push")

    # ---------------------------------------------------------------- server: apply
    def apply(self, ts: int, *, cached=None, wait_iters: int = 0, channel: int = 0, opt: Optional[OptimizerConfig] = None,
              stream=None):
        """F1b: apply push round ``ts`` from every alive source (into the table of ``channel``)."""
        cfg = self.cfg
        q = ts % cfg.ring

        def build():
            p = ApplyParams()
            p.S, p.inbox_cap, p.quant = self.S, cfg.inbox_cap, cfg.quant_code()
            p.table, p.mask = self.table_ptr(channel=channel), cfg.table_capacity - 1
            p.width, p.wide_vals = self.width, self.wide_vals_ptr(channel)
            p.key_begin, p.slot_mult = self.bounds_host[self.rank], self.slot_mult[self.rank]
            for r in range(self.S):
                p.inbox_keys[r] = self._inbox_keys(self.rank, q, r)
                p.inbox_vals[r] = self._inbox_vals(self.rank, q, r)
                p.ready[r] = self._ready(self.rank, q, r)
                p.count[r] = self._count(self.rank, q, r)
                p.mode[r] = self._mode(self.rank, q, r)
                p.alive[r] = 1 if self.alive[r] else 0
                p.slot_cache[r] = self._slot_cache_ptr(ts, r)
            p.stats, p.applied = ptr(self.push_stats), self._ctrl(self.rank, 0)
            p.bar, p.done, p.status = self._bar(2), self._done(2), ptr(self.status)
            if self.tile_off is not None:
                p.tile_off = self.tile_off[ts % self.tile_off.shape[0]].data_ptr()
                p.tiles, p.slow = self.tiles, self.sync_words.data_ptr() + 96
            return p
        p = self._params("apply", (q, channel), build)
        p.ts1, p.wait_iters = ts + 1, wait_iters
        for r in range(self.S):
            p.cached[r] = 1 if (cached is not None and cached[r]) else 0
        p.opt = (opt or self.opt).to_c()
        check(_lib.lib().psb_apply(C.byref(p), stream_ptr(stream)), "apply")
        self.applied_ts1 = ts + 1

    # ---------------------------------------------------------------- membership
    def _params(self, kind: str, key, build):
        """A fresh copy of the parameter block of ``kind`` whose round-independent part (peer
        addresses by ring slot, table, flags) ``build`` fills once per ``key``: with small requests the
        host would otherwise spend longer filling these blocks than the device spends on the kernels."""
        cache = self.__dict__.setdefault("_param_cache", {})
        tmpl = cache.get((kind, key))
        if tmpl is None:
            tmpl = cache[(kind, key)] = build()
        return type(tmpl).from_buffer_copy(tmpl)

    def set_alive(self, rank: int, alive: bool):
        """Host-side membership: a dead source is skipped by ``apply`` (its wait
        completes immediately), as with ``alive=false`` in the reference's
        ``Executor::RemoveNode`` (``system/executor.cc:303-313``)."""
        self.alive[rank] = alive
        self.__dict__.pop("_param_cache", None)        # the cached parameter blocks carry the membership

    def check_status(self, what: str = "data plane"):
        """Raise if a kernel of this plane reported an error; the plane's barrier and arrival words are
        cleared then, so that the next round can run (the stamps in the peers' flags are monotone and
        need no repair)."""
        _lib.check_status(self.status, what, reset=(self.sync_words,))

    # ---------------------------------------------------------------- model io
    def dump_nonzero(self):
        """(keys, w) of every entry with a non-zero weight, as CPU tensors sorted by key."""
        cap = self.cfg.table_capacity
        n = torch.zeros(1, dtype=torch.int64, device=self.device)
        # two passes: count, then fill
        L = _lib.lib()
        k0 = torch.empty(1, dtype=torch.int64, device=self.device)
        w0 = torch.empty(1, dtype=torch.float32, device=self.device)
        check(L.psb_table_dump(self.table_ptr(), cap, ptr(k0), ptr(w0), 0, ptr(n), stream_ptr()), "dump")
        cnt = int(n.item())
        keys = torch.empty(max(cnt, 1), dtype=torch.int64, device=self.device)
        w = torch.empty(max(cnt, 1), dtype=torch.float32, device=self.device)
        check(L.psb_table_dump(self.table_ptr(), cap, ptr(keys), ptr(w), cnt, ptr(n), stream_ptr()), "dump")
        keys, w = keys[:cnt].cpu(), w[:cnt].cpu()
        ukeys = keys.numpy().view("uint64")
        order = ukeys.argsort(kind="stable")
        return torch.from_numpy(ukeys[order].copy()), w[torch.from_numpy(order)]

    def export_state(self):
        """Every occupied slot: (keys uint64 numpy, s0, s1, w) for checkpoints."""
        cap = self.cfg.table_capacity
        L = _lib.lib()
        n = torch.zeros(1, dtype=torch.int64, device=self.device)
        d = torch.empty(1, dtype=torch.float32, device=self.device)
        k0 = torch.empty(1, dtype=torch.int64, device=self.device)
        check(L.psb_table_export(self.table_ptr(), cap, ptr(k0), ptr(d), ptr(d), ptr(d), 0, ptr(n), stream_ptr()), "export")
        cnt = int(n.item())
        keys = torch.empty(max(cnt, 1), dtype=torch.int64, device=self.device)
        s0, s1, w = (torch.empty(max(cnt, 1), dtype=torch.float32, device=self.device) for _ in range(3))
        check(L.psb_table_export(self.table_ptr(), cap, ptr(keys), ptr(s0), ptr(s1), ptr(w), cnt, ptr(n), stream_ptr()), "export")
        return keys[:cnt].cpu().numpy().view("uint64"), s0[:cnt].cpu(), s1[:cnt].cpu(), w[:cnt].cpu()

    def load_state(self, keys_u64, s0=None, s1=None, w=None):
        import numpy as np
        k = torch.from_numpy(np.ascontiguousarray(keys_u64).view("int64")).to(self.device)
        f = lambda t: None if t is None else t.to(self.device, torch.float32).contiguous()
        s0, s1, w = f(s0), f(s1), f(w)
        check(_lib.lib().psb_table_load(self.table_ptr(), self.cfg.table_capacity - 1, self.bounds_host[self.rank],
                                        self.slot_mult[self.rank], ptr(k), ptr(s0), ptr(s1),
                                        ptr(w), k.numel(), ptr(self.status), stream_ptr()), "load")
        torch.cuda.current_stream().synchronize()
