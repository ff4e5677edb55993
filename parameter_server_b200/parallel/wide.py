"""Wide-value shards: 64-wide bf16 vectors per key with fp32 AdaGrad accumulators.

The data plane mirrors :mod:`dataplane` (symmetric heap, per-(ring slot, source)
inboxes, release/acquire flags), with 128-byte value rows instead of scalars. The
pull is fused with the tensor-core product against the batch's context matrix
(``k_wide_pull_gemm``: tcgen05.mma, accumulator in TMEM, context matrix by TMA).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..ops import _lib
from ..ops._lib import MAX_SHARDS, check, ptr, stream_ptr
from ..utils.range import Range, shard_bounds
from .fabric import Fabric, HeapLayout

_vp, _u32, _u64, _i32, _f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float
WIDTH = 64


class _nullctx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class _PullArgs(C.Structure):
    _fields_ = [("S", _i32), ("N", _i32), ("keys", _vp * MAX_SHARDS), ("vals", _vp * MAX_SHARDS),
                ("mask", _u64 * MAX_SHARDS), ("key_begin", _u64 * MAX_SHARDS), ("slot_mult", _u64 * MAX_SHARDS),
                ("ukeys", _vp), ("n_unique", _vp), ("own_off", _vp), ("P", _vp), ("v_local", _vp), ("status", _vp),
                ("seg_off", _vp), ("csc_row", _vp), ("row_ctx", _vp), ("margin", _vp),
                ("plong_n", _vp), ("plong_list", _vp), ("plong_rows", _vp), ("plong_cap", _u32)]


class _PushArgs(C.Structure):
    _fields_ = [("S", _i32), ("N", _i32), ("ts1", _u32), ("inbox_cap", _u32),
                ("inbox_keys", _vp * MAX_SHARDS), ("inbox_vals", _vp * MAX_SHARDS),
                ("ready", _vp * MAX_SHARDS), ("count", _vp * MAX_SHARDS),
                ("ukeys", _vp), ("n_unique", _vp), ("own_off", _vp), ("seg_off", _vp), ("csc_row", _vp),
                ("gcoef", _vp), ("row_ctx", _vp), ("ctx", _vp), ("done", _vp), ("status", _vp),
                ("bar", _vp), ("n_long", _vp), ("long_list", _vp), ("long_acc", _vp), ("long_cap", _u32)]


class _ApplyArgs(C.Structure):
    _fields_ = [("S", _i32), ("ts1", _u32), ("inbox_cap", _u32), ("keys", _vp), ("vals", _vp), ("acc", _vp),
                ("mask", _u64), ("key_begin", _u64), ("slot_mult", _u64),
                ("inbox_keys", _vp * MAX_SHARDS), ("inbox_vals", _vp * MAX_SHARDS),
                ("ready", _vp * MAX_SHARDS), ("count", _vp * MAX_SHARDS), ("alive", C.c_uint8 * MAX_SHARDS),
                ("alpha", _f32), ("beta", _f32), ("wait_iters", _u32),
                ("applied", _vp), ("bar", _vp), ("done", _vp), ("status", _vp)]


class _XArgs(C.Structure):
    _fields_ = [("S", _i32), ("me", _i32), ("N", _i32), ("ts1", _u32), ("req_cap", _u32), ("wait_iters", _u32), ("phases", _u32),
                ("keys", _vp), ("vals", _vp), ("mask", _u64), ("key_begin", _u64), ("slot_mult", _u64),
                ("req_keys", _vp * MAX_SHARDS), ("req_hdr", _vp * MAX_SHARDS), ("req_ready", _vp * MAX_SHARDS),
                ("my_resp_ready", _vp * MAX_SHARDS), ("my_resp_rows", _vp),
                ("my_req_keys", _vp * MAX_SHARDS), ("my_req_hdr", _vp * MAX_SHARDS), ("my_req_ready", _vp * MAX_SHARDS),
                ("resp_rows", _vp * MAX_SHARDS), ("resp_ready", _vp * MAX_SHARDS), ("alive", C.c_uint8 * MAX_SHARDS),
                ("ukeys", _vp), ("n_unique", _vp), ("own_off", _vp), ("P", _vp), ("done", _vp), ("status", _vp),
                ("seg_off", _vp), ("csc_row", _vp), ("row_ctx", _vp), ("margin", _vp),
                ("plong_n", _vp), ("plong_list", _vp), ("plong_rows", _vp), ("plong_cap", _u32)]


def _declare():
    L = _lib.lib()
    if getattr(L, "_wide_declared", False):
        return L
    L.psb_wide_init.argtypes = [_vp, _vp, _vp, _u64, _vp]
    L.psb_wide_load.argtypes = [_vp, _vp, _u64, _u64, _u64, _vp, _vp, _u32, _vp, _vp]
    L.psb_wide_pull_gemm.argtypes = [_vp, _vp, _u32, _vp]
    L.psb_wide_pull_xgemm.argtypes = [_vp, _vp, _u32, _vp]
    L.psb_wide_rowsum.argtypes = [_vp, _i32, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]
    L.psb_wide_rowloss.argtypes = [_vp, _vp, _u32, _vp, _vp, _vp, _vp, _vp, _u32, _i32, _vp, _vp, _vp]
    L.psb_wide_push.argtypes = [_vp, _vp]
    L.psb_wide_apply.argtypes = [_vp, _vp]
    L.psb_wide_args_size.argtypes = [_i32]
    for i, st in enumerate((_PullArgs, _PushArgs, _ApplyArgs, _XArgs)):
        if L.psb_wide_args_size(i) != C.sizeof(st):
            raise RuntimeError(f"{st.__name__}: binding is {C.sizeof(st)} bytes, library expects {L.psb_wide_args_size(i)}")
    L._wide_declared = True
    return L


@dataclass
class WideConfig:
    table_capacity: int              # slots per shard (power of two)
    inbox_cap: int                   # records per (owner, source) inbox
    ring: int = 2
    alpha: float = 0.05              # AdaGrad: eta = alpha / (sqrt(sum g^2) + beta)
    beta: float = 1.0
    key_range: Range = field(default_factory=Range.all)
    ordered_slots: bool = True
    pull_cap: int = 0                # > 0: exchange pull (keys to the owners, rows back, in bulk); unique keys per batch


def wide_layout(cfg: WideConfig, world: int) -> HeapLayout:
    assert cfg.table_capacity & (cfg.table_capacity - 1) == 0
    lay = HeapLayout(align=1024)
    lay.add("ctrl", 4096)
    lay.add("keys", cfg.table_capacity * 8)
    lay.add("vals", cfg.table_capacity * WIDTH * 2)
    lay.add("acc", cfg.table_capacity * WIDTH * 4)
    lay.add("inbox_keys", cfg.ring * world * cfg.inbox_cap * 8)
    lay.add("inbox_vals", cfg.ring * world * cfg.inbox_cap * WIDTH * 2)
    if cfg.pull_cap:
        lay.add("xctrl", 4096)                                    # flags and headers of the exchange pull
        lay.add("req_keys", 2 * world * cfg.inbox_cap * 8)        # [parity][source][key]
        lay.add("resp_rows", 2 * cfg.pull_cap * WIDTH * 2)        # [parity][unique key][64] bf16
    return lay


class WidePlane:
    """One wide shard + worker endpoint."""

    def __init__(self, fabric: Fabric, cfg: WideConfig):
        self.L = _declare()
        self.fabric, self.cfg = fabric, cfg
        self.rank, self.S = fabric.rank, fabric.world
        self.lay = wide_layout(cfg, self.S)
        assert self.lay.total() <= fabric.heap_bytes
        dev = fabric.device
        self.device = dev
        self.bounds_host = shard_bounds(cfg.key_range, self.S)
        self.bounds = torch.tensor([b if b < (1 << 63) else b - (1 << 64) for b in self.bounds_host], dtype=torch.int64, device=dev)
        self.slot_mult = []
        for s in range(self.S):
            size = self.bounds_host[s + 1] - self.bounds_host[s]
            m = (cfg.table_capacity << 64) // size if (cfg.ordered_slots and size > cfg.table_capacity) else 0
            self.slot_mult.append(m if m < (1 << 64) else 0)
        self.sync = torch.zeros(16, dtype=torch.int32, device=dev)
        # scratch of the push for keys with very long segments (zeroed once, left zeroed by the kernel)
        self.long_cap = max(64, cfg.inbox_cap // 256 + 1)
        self.long_list = torch.zeros(self.long_cap * 4, dtype=torch.int32, device=dev)   # {key, first chunk, begin, end}
        self.long_acc = torch.zeros(self.long_cap * WIDTH, dtype=torch.float32, device=dev)
        # the fused pull's list of keys with long segments: {count, chunks}, entries, their rows of products
        self.plong_cap = max(64, cfg.inbox_cap // 512 + 1)
        self.plong_n = torch.zeros(1, dtype=torch.int64, device=dev)
        self.plong_list = torch.zeros(self.plong_cap * 4, dtype=torch.int32, device=dev)
        self.plong_rows = torch.zeros(self.plong_cap * 128, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stats = torch.zeros(4, dtype=torch.float64, device=dev)
        check(self.L.psb_wide_init(self._p("keys"), self._p("vals"), self._p("acc"), cfg.table_capacity, stream_ptr()), "wide_init")

    def _p(self, name, rank=None, off=0):
        return self.fabric.ptr(self.rank if rank is None else rank, self.lay[name] + off)

    def _ctrl(self, rank, word):
        return self._p("ctrl", rank, 4 * word)

    def _ready(self, owner, q, src):
        return self._ctrl(owner, 8 + q * self.S + src)

    def _count(self, owner, q, src):
        return self._ctrl(owner, 8 + self.cfg.ring * self.S + q * self.S + src)

    def _ik(self, owner, q, src):
        return self._p("inbox_keys", owner, ((q * self.S + src) * self.cfg.inbox_cap) * 8)

    def _iv(self, owner, q, src):
        return self._p("inbox_vals", owner, ((q * self.S + src) * self.cfg.inbox_cap) * WIDTH * 2)

    def load(self, keys_u64: np.ndarray, rows: torch.Tensor):
        """Insert (key, 64-value row) pairs that belong to this shard."""
        k = torch.from_numpy(np.ascontiguousarray(keys_u64).view(np.int64)).to(self.device)
        v = rows.to(self.device, torch.bfloat16).contiguous()
        check(self.L.psb_wide_load(self._p("keys"), self._p("vals"), self.cfg.table_capacity - 1, self.bounds_host[self.rank],
                                   self.slot_mult[self.rank], ptr(k), ptr(v), k.numel(), ptr(self.status), stream_ptr()), "wide_load")
        torch.cuda.current_stream().synchronize()

    def _xflag(self, rank, kind, par, peer):
        """Exchange flag word: kind 0 = request ready, 1 = response ready."""
        return self._p("xctrl", rank, 4 * ((kind * 2 + par) * self.S + peer))

    def _xhdr(self, rank, par, peer):
        return self._p("xctrl", rank, 4 * (4 * self.S + (par * self.S + peer) * 2))

    def _fused(self, a, b, P, fuse_margins: bool, row_ctx, stream):
        """``fuse_margins``: the kernel adds every product a row needs into ``b.margin`` (zeroed here) and
        ``P`` may be None; :meth:`rowloss` then finishes the rows."""
        a.P = ptr(P)
        if fuse_margins:
            with torch.cuda.stream(stream) if stream is not None else _nullctx():
                b.margin[:max(1, b.n_rows)].zero_()
            a.seg_off, a.csc_row, a.row_ctx, a.margin = ptr(b.seg_off), ptr(b.csc_row), ptr(row_ctx), ptr(b.margin)
            a.plong_n, a.plong_list, a.plong_rows = ptr(self.plong_n), ptr(self.plong_list), ptr(self.plong_rows)
            a.plong_cap = self.plong_cap
            self._fused_call = (a.N, row_ctx)
        else:
            assert P is not None

    def pull_xgemm(self, b, ctx: torch.Tensor, P: Optional[torch.Tensor], ts: int, *, phases: int = 7, wait_iters: int = 0,
                   fuse_margins: bool = False, row_ctx: Optional[torch.Tensor] = None, stream=None):
        """Exchange form of :meth:`pull_gemm` for round ``ts`` (every rank calls it every round):
        keys to the owners in bulk, value rows back in bulk, the product on the local copy."""
        cfg = self.cfg
        assert cfg.pull_cap >= b.max_nnz and 4 * (4 * self.S + 4 * self.S) <= 4096
        assert ctx.dtype == torch.bfloat16 and ctx.is_contiguous() and ctx.shape[1] == WIDTH
        par = ts & 1
        a = _XArgs()
        a.S, a.me, a.N, a.ts1, a.req_cap, a.wait_iters, a.phases = self.S, self.rank, ctx.shape[0], ts + 1, cfg.inbox_cap, wait_iters, phases
        a.keys, a.vals = self._p("keys"), self._p("vals")
        a.mask, a.key_begin, a.slot_mult = cfg.table_capacity - 1, self.bounds_host[self.rank], self.slot_mult[self.rank]
        rb = cfg.inbox_cap * 8
        for s in range(self.S):
            a.req_keys[s] = self._p("req_keys", s, (par * self.S + self.rank) * rb)
            a.req_hdr[s], a.req_ready[s] = self._xhdr(s, par, self.rank), self._xflag(s, 0, par, self.rank)
            a.my_resp_ready[s] = self._xflag(self.rank, 1, par, s)
            a.my_req_keys[s] = self._p("req_keys", self.rank, (par * self.S + s) * rb)
            a.my_req_hdr[s], a.my_req_ready[s] = self._xhdr(self.rank, par, s), self._xflag(self.rank, 0, par, s)
            a.resp_rows[s] = self._p("resp_rows", s, par * cfg.pull_cap * WIDTH * 2)
            a.resp_ready[s] = self._xflag(s, 1, par, self.rank)
            a.alive[s] = 1
        a.my_resp_rows = self._p("resp_rows", self.rank, par * cfg.pull_cap * WIDTH * 2)
        a.ukeys, a.n_unique, a.own_off = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off)
        a.done, a.status = self.sync.data_ptr() + 48, ptr(self.status)
        self._fused(a, b, P, fuse_margins and bool(phases & 4), row_ctx, stream)
        check(self.L.psb_wide_pull_xgemm(C.byref(a), ptr(ctx), b.max_nnz, stream_ptr(stream)), "wide_pull_xgemm")

    def pulled_rows(self, ts: int, n: int) -> torch.Tensor:
        """The value rows this worker received in the exchange of round ``ts`` ([n, 64] bf16)."""
        return self.fabric.view(self.lay["resp_rows"] + (ts & 1) * self.cfg.pull_cap * WIDTH * 2, (n, WIDTH), torch.bfloat16)

    def pull_gemm(self, b, ctx: torch.Tensor, P: Optional[torch.Tensor], v_local: Optional[torch.Tensor] = None,
                  fuse_margins: bool = False, row_ctx: Optional[torch.Tensor] = None, stream=None):
        """``P[u, n] = <value row of unique key u, ctx[n]>`` for the batch ``b``.
        ``ctx``: [N, 64] bf16 with N in (64, 128)."""
        a = _PullArgs()
        a.S, a.N = self.S, ctx.shape[0]
        for s in range(self.S):
            a.keys[s], a.vals[s] = self._p("keys", s), self._p("vals", s)
            a.mask[s], a.key_begin[s], a.slot_mult[s] = self.cfg.table_capacity - 1, self.bounds_host[s], self.slot_mult[s]
        a.ukeys, a.n_unique, a.own_off = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off)
        a.v_local, a.status = ptr(v_local), ptr(self.status)
        self._fused(a, b, P, fuse_margins, row_ctx, stream)
        assert ctx.dtype == torch.bfloat16 and ctx.is_contiguous() and ctx.shape[1] == WIDTH
        check(self.L.psb_wide_pull_gemm(C.byref(a), ptr(ctx), b.max_nnz, stream_ptr(stream)), "wide_pull_gemm")

    def rowsum(self, b, P: torch.Tensor, N: int, row_ctx: Optional[torch.Tensor] = None, stream=None):
        check(self.L.psb_wide_rowsum(ptr(P), N, ptr(b.row_ptr), b.n_rows, b.fixed_z, ptr(b.csr_col), ptr(row_ctx), ptr(b.y),
                                     ptr(b.gcoef), ptr(b.margin), ptr(self.stats), stream_ptr(stream)), "wide_rowsum")

    def rowloss(self, b, stream=None):
        """Loss, accuracy counters and ``gcoef`` from the margins that a fused pull accumulated."""
        N, row_ctx = self._fused_call
        check(self.L.psb_wide_rowloss(ptr(b.margin), ptr(b.y), b.n_rows, ptr(b.gcoef), ptr(self.stats), ptr(self.plong_n),
                                      ptr(self.plong_list), ptr(self.plong_rows), self.plong_cap, N, ptr(b.csc_row),
                                      ptr(row_ctx), stream_ptr(stream)), "wide_rowloss", kernels=2)

    def push(self, b, ctx: torch.Tensor, ts: int, row_ctx: Optional[torch.Tensor] = None, stream=None):
        q = ts % self.cfg.ring
        a = _PushArgs()
        a.S, a.N, a.ts1, a.inbox_cap = self.S, ctx.shape[0], ts + 1, self.cfg.inbox_cap
        for s in range(self.S):
            a.inbox_keys[s], a.inbox_vals[s] = self._ik(s, q, self.rank), self._iv(s, q, self.rank)
            a.ready[s], a.count[s] = self._ready(s, q, self.rank), self._count(s, q, self.rank)
        a.ukeys, a.n_unique, a.own_off = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off)
        a.seg_off, a.csc_row, a.gcoef, a.row_ctx, a.ctx = ptr(b.seg_off), ptr(b.csc_row), ptr(b.gcoef), ptr(row_ctx), ptr(ctx)
        a.done, a.status = self.sync.data_ptr() + 8, ptr(self.status)
        a.bar, a.n_long = self.sync.data_ptr() + 32, self.sync.data_ptr() + 40
        a.long_list, a.long_acc, a.long_cap = ptr(self.long_list), ptr(self.long_acc), self.long_cap
        check(self.L.psb_wide_push(C.byref(a), stream_ptr(stream)), "wide_push")

    def apply(self, ts: int, wait_iters: int = 0, stream=None):
        q = ts % self.cfg.ring
        a = _ApplyArgs()
        a.S, a.ts1, a.inbox_cap = self.S, ts + 1, self.cfg.inbox_cap
        a.keys, a.vals, a.acc = self._p("keys"), self._p("vals"), self._p("acc")
        a.mask, a.key_begin, a.slot_mult = self.cfg.table_capacity - 1, self.bounds_host[self.rank], self.slot_mult[self.rank]
        for r in range(self.S):
            a.inbox_keys[r], a.inbox_vals[r] = self._ik(self.rank, q, r), self._iv(self.rank, q, r)
            a.ready[r], a.count[r], a.alive[r] = self._ready(self.rank, q, r), self._count(self.rank, q, r), 1
        a.alpha, a.beta, a.wait_iters = self.cfg.alpha, self.cfg.beta, wait_iters
        a.applied, a.bar, a.done, a.status = self._ctrl(self.rank, 0), self.sync.data_ptr() + 16, self.sync.data_ptr() + 24, ptr(self.status)
        check(self.L.psb_wide_apply(C.byref(a), stream_ptr(stream)), "wide_apply")

    def lookup(self, keys_u64: np.ndarray) -> torch.Tensor:
        """Rows of ``keys`` owned by this shard (zeros if absent), for tests and dumps."""
        cap = self.cfg.table_capacity
        tk = self.fabric.view(self.lay["keys"], (cap,), torch.int64).cpu().numpy().view(np.uint64)
        tv = self.fabric.view(self.lay["vals"], (cap, WIDTH), torch.bfloat16).cpu()
        pos = {int(k): i for i, k in enumerate(tk.tolist()) if k != (1 << 64) - 1}
        out = torch.zeros(len(keys_u64), WIDTH, dtype=torch.bfloat16)
        for i, k in enumerate(keys_u64.tolist()):
            j = pos.get(int(k))
            if j is not None:
                out[i] = tv[j]
        return out

    def check_status(self, what="wide plane"):
        _lib.check_status(self.status, what, reset=(self.sync,))
