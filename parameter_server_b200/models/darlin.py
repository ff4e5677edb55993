"""Darlin on the GPUs: delayed block proximal gradient (block coordinate descent)
for L1-regularised logistic regression.

Every rank is a worker (its rows, CSC over its unique keys) and an owner (a
contiguous range of the global column space = the sorted union of all keys,
cut at the shards' key-range boundaries). Per feature block three fused kernels
run on every rank (``csrc/cuda/darlin.cu``): gradient + reduce-to-owner,
owner update + broadcast, margin update. Blocks are pipelined with bounded
delay ``tau``: the gradients of block ``t + tau`` are computed before the
weights of block ``t`` have been applied, which is the device form of the
scheduler's ``wait_time`` window (``app/linear_method/darlin.h:157-164``).

The pass structure, KKT-filter threshold rule and stopping test follow
``DarlinScheduler::Run`` (``app/linear_method/darlin.h:21-132``).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import _lib
from ..ops._lib import DarlinDual, DarlinGrad, DarlinPass, DarlinUpdate, check, ptr, stream_ptr
from ..ops.localize import LocalBatch
from ..parallel.fabric import Fabric, HeapLayout
from ..utils.range import Range, shard_bounds


@dataclass
class DarlinConfig:
    lambda_l1: float = 1.0
    eta: float = 0.9                 # learning_rate.alpha
    delta_init: float = 1.0
    delta_max: float = 5.0
    kkt_ratio: float = 10.0
    max_pass: int = 10
    epsilon: float = 1e-4
    block_cols: int = 1 << 16        # columns per feature block
    tau: int = 0                     # max_block_delay
    random_block_order: bool = True
    key_range: Range = Range.all()


def darlin_heap_bytes(cfg: DarlinConfig, world: int) -> int:
    return _layout(cfg, world).total()


def _layout(cfg: DarlinConfig, world: int) -> HeapLayout:
    R = cfg.tau + 2
    lay = HeapLayout()
    lay.add("flags", 4 * 2 * R * world + 64)                 # gu_ready[R][src], wnew_ready[R][owner]
    lay.add("gu_inbox", R * world * 2 * cfg.block_cols * 4)   # [R][src][2][block]
    lay.add("wnew", R * cfg.block_cols * 4)                   # [R][block]
    return lay


class DarlinRank:
    """Worker + owner state of one rank."""

    def __init__(self, fabric: Fabric, cfg: DarlinConfig, keys: torch.Tensor, y: torch.Tensor, *, fixed_z: int = 0,
                 row_ptr: Optional[torch.Tensor] = None, vals: Optional[torch.Tensor] = None,
                 global_keys: Optional[torch.Tensor] = None):
        """``keys``: per-nonzero uint64 keys (int64 view) of this rank's rows in CSR
        order; ``global_keys``: sorted union of every rank's unique keys (if None,
        this rank's own unique keys -- single-rank use)."""
        self.fabric, self.cfg = fabric, cfg
        self.rank, self.S = fabric.rank, fabric.world
        dev = fabric.device
        self.dev = dev
        self.lay = _layout(cfg, self.S)
        assert self.lay.total() <= fabric.heap_bytes
        self.R = cfg.tau + 2
        nnz = keys.numel()
        self.n_rows = y.numel()
        self.y = y.contiguous().float()
        # CSC of the local rows: the same sort + localise as a minibatch, once
        self.b = LocalBatch(self.n_rows, nnz, 1, dev, real_values=vals is not None)
        bounds1 = torch.tensor([0, -1], dtype=torch.int64, device=dev)
        self.b.localize(keys, self.y, bounds1, fixed_z=fixed_z, row_ptr=row_ptr, vals=vals, hash_seed=None)
        torch.cuda.synchronize(dev)
        self.U = int(self.b.n_unique.item())
        self.local_keys = self.b.ukeys[:self.U]
        self.set_global_keys(self.local_keys if global_keys is None else global_keys)
        self.margin = torch.zeros(self.n_rows, dtype=torch.float32, device=dev)
        self.sync = torch.zeros(16, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.violation = torch.zeros(1, dtype=torch.float32, device=dev)
        self.stage = torch.zeros(self.R * 2 * cfg.block_cols, dtype=torch.float32, device=dev)   # one area per ring slot
        self.kkt_threshold = 1e20
        self.step = 0
        self.phase_ns: Optional[torch.Tensor] = None   # int64[4]: set to have run_pass add up its phase times

    def set_global_keys(self, global_keys: torch.Tensor):
        """``global_keys``: the sorted global key list (uint64 as int64, on the device). The local keys'
        columns and the shards' column ranges are found on the device (binary searches over the list)."""
        cfg, dev = self.cfg, self.dev
        self.global_keys = global_keys
        self.n_cols = global_keys.numel()
        sign = -(1 << 63)                                 # signed order of (k ^ sign) = unsigned order of k
        gk = global_keys ^ sign
        gcol = torch.searchsorted(gk, self.local_keys ^ sign)
        self.gcol = gcol.to(torch.int32)
        self.gcol_host = gcol.cpu().numpy()               # block -> local key range look-ups on the host
        # the global column of every nonzero (CSC order): 4 bytes per nonzero that save the block kernels
        # two dependent gathers per nonzero (word base -> local key -> column)
        U = self.local_keys.numel()
        seg = self.b.seg_off[:U + 1].long()
        self.csc_col = torch.repeat_interleave(self.gcol, seg[1:] - seg[:-1]) if U else torch.zeros(0, dtype=torch.int32, device=dev)
        self.seg_host = seg.cpu().numpy() if U else np.zeros(1, dtype=np.int64)      # the blocks' nonzero ranges go into their parameter blocks
        bh = shard_bounds(cfg.key_range, self.S)
        edges = torch.from_numpy(np.array([min(b, (1 << 64) - 1) for b in bh[:-1]], dtype=np.uint64).view(np.int64)).to(dev) ^ sign
        self.shard_col = torch.searchsorted(gk, edges).tolist() + [self.n_cols]
        f32 = torch.float32
        n = max(1, self.n_cols)
        # owner state (only my column range is touched) and worker copies
        self.w_own = torch.zeros(n, dtype=f32, device=dev)
        self.delta_own = torch.full((n,), cfg.delta_init, dtype=f32, device=dev)
        self.active_own = torch.ones(n, dtype=torch.uint8, device=dev)
        self.w_cur = torch.zeros(n, dtype=f32, device=dev)
        self.delta_w = torch.full((n,), cfg.delta_init, dtype=f32, device=dev)
        self.active_w = torch.ones(n, dtype=torch.uint8, device=dev)
        nb = (self.n_cols + cfg.block_cols - 1) // cfg.block_cols
        self.blocks = [(i * cfg.block_cols, min(self.n_cols, (i + 1) * cfg.block_cols)) for i in range(nb)]
        self.prior_blocks: List[int] = []

    def set_initial_weights(self, w0: torch.Tensor):
        """Start from ``w0`` (float32 per global column, the same vector on every rank) instead of zero: the
        owners' weights and the workers' copies take it, and the margins become X w0 over this rank's rows
        (the reference's ``init_w``: servers allocate with it, ``learner/bcd.h:199``, workers compute
        ``X w`` from the first pull, ``learner/bcd.h:414-416``). Call before the first pass."""
        n = self.n_cols
        w0 = w0.to(self.dev, torch.float32).flatten()
        assert w0.numel() == n
        self.w_own[:n].copy_(w0)
        self.w_cur[:n].copy_(w0)
        self.margin.zero_()
        nnz = self.csc_col.numel()
        if nnz:
            contrib = w0[self.csc_col.long()]
            if self.b.csc_val is not None:
                contrib = contrib * self.b.csc_val[:nnz]
            self.margin.index_add_(0, self.b.csc_row[:nnz].long(), contrib)
        torch.cuda.current_stream(self.dev).synchronize()      # the passes run on streams of their own

    def set_blocks(self, blocks: List[tuple], prior: Optional[List[int]] = None):
        """Use the given column ranges as feature blocks (none wider than ``cfg.block_cols``); ``prior``
        lists block indices that open the first pass, one after another (no delay)."""
        assert all(0 <= c0 < c1 <= self.n_cols and c1 - c0 <= self.cfg.block_cols for c0, c1 in blocks)
        self.blocks = list(blocks)
        self.prior_blocks = list(prior or [])
        self.__dict__.pop("_param_cache", None)
        self.__dict__.pop("_pass_dev", None)

    # ---- addresses in a rank's heap
    def _flag(self, rank: int, kind: int, q: int, idx: int) -> int:
        return self.fabric.ptr(rank, self.lay["flags"] + 4 * ((kind * self.R + q) * self.S + idx))

    def _gu(self, owner: int, q: int, src: int) -> int:
        return self.fabric.ptr(owner, self.lay["gu_inbox"] + ((q * self.S + src) * 2 * self.cfg.block_cols) * 4)

    def _wnew(self, rank: int, q: int) -> int:
        return self.fabric.ptr(rank, self.lay["wnew"] + q * self.cfg.block_cols * 4)

    def _block_u(self, c0: int, c1: int):
        return int(np.searchsorted(self.gcol_host, c0)), int(np.searchsorted(self.gcol_host, c1))

    # ---- the three kernels of a block
    def streams(self):
        """(gradient stream, update + dual stream) of the two-stream block pipeline."""
        if "_streams" not in self.__dict__:
            self._streams = (torch.cuda.Stream(device=self.dev), torch.cuda.Stream(device=self.dev))
        return self._streams

    def _cached(self, kind: str, blk: int, q: int):
        """Parameter blocks are built once per (kernel, block, ring slot): with hundreds of
        blocks per pass the launches are otherwise bound by the host filling these structs."""
        cache = self.__dict__.setdefault("_param_cache", {})
        return cache, (kind, blk, q), cache.get((kind, blk, q))

    def _grad_params(self, blk: int, q: int) -> DarlinGrad:
        cache, key, p = self._cached("grad", blk, q)
        if p is not None:
            return p
        c0, c1 = self.blocks[blk]
        u0, u1 = self._block_u(c0, c1)
        p = cache[key] = DarlinGrad()
        p.S, p.c0, p.c1, p.u0, p.u1, p.block_cap = self.S, c0, c1, u0, u1, self.cfg.block_cols
        for s in range(self.S + 1):
            p.shard_col[s] = self.shard_col[s]
        b = self.b
        p.seg_off, p.csc_row, p.csc_val = ptr(b.seg_off), ptr(b.csc_row), ptr(b.csc_val)
        p.flagbits, p.wordbase, p.gcol = ptr(b.flagbits), ptr(b.wordbase), ptr(self.gcol)
        p.y, p.margin, p.active, p.delta, p.stage = ptr(self.y), ptr(self.margin), ptr(self.active_w), ptr(self.delta_w), self.stage.data_ptr() + q * 2 * self.cfg.block_cols * 4
        for s in range(self.S):
            p.gu_inbox[s] = self._gu(s, q, self.rank)
            p.ready[s] = self._flag(s, 0, q, self.rank)
        p.bar, p.done, p.status = self.sync.data_ptr(), self.sync.data_ptr() + 8, ptr(self.status)
        p.csc_col = ptr(self.csc_col) if self.csc_col.numel() else None
        p.nz0, p.nz1 = int(self.seg_host[u0]), int(self.seg_host[u1])
        return p

    def _update_params(self, blk: int, q: int):
        """The owner's parameter block, or False when none of the block's columns is mine."""
        cache, key, p = self._cached("update", blk, q)
        if p is not None:
            return p
        c0, c1 = self.blocks[blk]
        my0, my1 = max(c0, self.shard_col[self.rank]), min(c1, self.shard_col[self.rank + 1])
        if my1 <= my0:
            cache[key] = False
            return False
        p = cache[key] = DarlinUpdate()
        p.S, p.c0, p.c1, p.my0, p.my1, p.block_cap = self.S, c0, c1, my0, my1, self.cfg.block_cols
        for r in range(self.S):
            p.gu_inbox[r] = self._gu(self.rank, q, r)
            p.ready[r] = self._flag(self.rank, 0, q, r)
            p.alive[r] = 1
            p.wnew_inbox[r] = self._wnew(r, q)
            p.wnew_ready[r] = self._flag(r, 1, q, self.rank)
        p.w, p.delta, p.active = ptr(self.w_own), ptr(self.delta_own), ptr(self.active_own)
        cfg = self.cfg
        p.eta, p.lam, p.delta_max = cfg.eta, cfg.lambda_l1, cfg.delta_max
        p.violation = ptr(self.violation)
        p.done, p.status = self.sync.data_ptr() + 24, ptr(self.status)
        return p

    def _dual_params(self, blk: int, q: int) -> DarlinDual:
        cache, key, p = self._cached("dual", blk, q)
        if p is not None:
            return p
        c0, c1 = self.blocks[blk]
        u0, u1 = self._block_u(c0, c1)
        p = cache[key] = DarlinDual()
        p.S, p.c0, p.c1, p.u0, p.u1, p.block_cap = self.S, c0, c1, u0, u1, self.cfg.block_cols
        for s in range(self.S + 1):
            p.shard_col[s] = self.shard_col[s]
        b = self.b
        p.seg_off, p.csc_row, p.csc_val = ptr(b.seg_off), ptr(b.csc_row), ptr(b.csc_val)
        p.flagbits, p.wordbase, p.gcol = ptr(b.flagbits), ptr(b.wordbase), ptr(self.gcol)
        p.margin, p.w_cur, p.delta, p.active = ptr(self.margin), ptr(self.w_cur), ptr(self.delta_w), ptr(self.active_w)
        p.delta_max, p.wnew = self.cfg.delta_max, self._wnew(self.rank, q)
        for s in range(self.S):
            p.wnew_ready[s] = self._flag(self.rank, 1, q, s)
            p.alive[s] = 1
        p.bar, p.status = self.sync.data_ptr() + 32, ptr(self.status)
        p.csc_col = ptr(self.csc_col) if self.csc_col.numel() else None
        p.nz0, p.nz1 = int(self.seg_host[u0]), int(self.seg_host[u1])
        return p

    def grad(self, blk: int, ts: int, stream=None):
        p = self._grad_params(blk, ts % self.R)
        p.ts1 = ts + 1
        check(_lib.lib().psb_darlin_grad(C.byref(p), stream_ptr(stream)), "darlin_grad")

    def update(self, blk: int, ts: int, wait_iters: int = 0, stream=None):
        p = self._update_params(blk, ts % self.R)
        if p is False:
            return                                    # no column of this block is mine
        p.ts1, p.kkt_threshold, p.wait_iters = ts + 1, self.kkt_threshold, wait_iters
        check(_lib.lib().psb_darlin_update(C.byref(p), stream_ptr(stream)), "darlin_update")

    def dual(self, blk: int, ts: int, wait_iters: int = 0, stream=None):
        p = self._dual_params(blk, ts % self.R)
        p.ts1, p.wait_iters = ts + 1, wait_iters
        check(_lib.lib().psb_darlin_dual(C.byref(p), stream_ptr(stream)), "darlin_dual")

    # ---- a whole pass in one launch
    def _pass_arrays(self):
        """Device copies of every block's parameter blocks, [block * R + ring slot] (built once)."""
        arr = self.__dict__.get("_pass_dev")
        if arr is not None:
            return arr
        nb, R = len(self.blocks), self.R
        G, U, D = (DarlinGrad * (nb * R))(), (DarlinUpdate * (nb * R))(), (DarlinDual * (nb * R))()
        for blk in range(nb):
            for q in range(R):
                C.memmove(C.byref(G, (blk * R + q) * C.sizeof(DarlinGrad)), C.byref(self._grad_params(blk, q)), C.sizeof(DarlinGrad))
                u = self._update_params(blk, q)
                if u is not False:
                    C.memmove(C.byref(U, (blk * R + q) * C.sizeof(DarlinUpdate)), C.byref(u), C.sizeof(DarlinUpdate))
                C.memmove(C.byref(D, (blk * R + q) * C.sizeof(DarlinDual)), C.byref(self._dual_params(blk, q)), C.sizeof(DarlinDual))

        def to_dev(a):
            return torch.frombuffer(bytearray(bytes(a)), dtype=torch.uint8).to(self.dev)
        arr = self._pass_dev = (to_dev(G), to_dev(U), to_dev(D))
        self._pass_bar = torch.zeros(4, dtype=torch.int32, device=self.dev)
        return arr

    def run_pass(self, order: Sequence[int], ts_base: int, tau: int, wait_iters: int = 0, stream=None):
        """All blocks of ``order`` with stamps ``ts_base ..`` in ONE cooperative launch: gradients run
        ``tau`` blocks ahead of the weight application (``k_darlin_pass``). Only for one rank per GPU:
        ranks that share a GPU would wait for each other's launches."""
        G, U, D = self._pass_arrays()
        p = DarlinPass()
        od = torch.tensor(list(order), dtype=torch.int32, device=self.dev)
        p.grad, p.update, p.dual, p.order = ptr(G), ptr(U), ptr(D), ptr(od)
        p.n_steps, p.ts_base, p.tau, p.ring = len(order), ts_base, tau, self.R
        p.kkt_threshold, p.wait_iters = self.kkt_threshold, wait_iters
        p.bar, p.status = ptr(self._pass_bar), ptr(self.status)
        p.phase_ns = ptr(self.phase_ns) if self.phase_ns is not None else None
        check(_lib.lib().psb_darlin_pass(C.byref(p), stream_ptr(stream)), "darlin_pass")
        self._pass_order = od          # keep the schedule alive until the launch has run

    def reset_kkt_filter(self):
        self.active_own.fill_(1)
        self.active_w.fill_(1)

    def evaluate(self):
        """(loss over my rows, lambda*|w|_1 / nnz / active over my columns, max violation)."""
        out = torch.zeros(4, dtype=torch.float64, device=self.dev)
        c0, c1 = self.shard_col[self.rank], self.shard_col[self.rank + 1]
        check(_lib.lib().psb_darlin_eval(ptr(self.y), ptr(self.margin), self.n_rows, ptr(self.w_own), ptr(self.active_own),
                                         c0, c1, self.cfg.lambda_l1, ptr(out), stream_ptr()), "darlin_eval")
        vals = out.tolist() + [float(self.violation.item())]
        self.violation.zero_()
        return vals

    def my_model(self):
        """(keys uint64, w) of my non-zero weights."""
        c0, c1 = self.shard_col[self.rank], self.shard_col[self.rank + 1]
        w = self.w_own[c0:c1]
        nz = torch.nonzero((w != 0) & (w == w)).flatten()
        return self.global_keys[c0:c1][nz].cpu().numpy().view(np.uint64), w[nz].cpu().numpy()

    def check_status(self, what="darlin"):
        _lib.check_status(self.status, what, reset=(self.sync, self.__dict__.get("_pass_bar")))


def run_darlin(ranks: Sequence[DarlinRank], *, all_reduce=None, verbose: bool = False, num_examples: Optional[int] = None,
               save_every: int = 0, save_fn=None):
    """Drive passes over the blocks. ``ranks``: every rank of an emulated fabric
    (kernels of the ranks run one after another), or the single local rank of a
    multi-process run, with ``all_reduce(values, op)`` combining the per-pass
    scalars across processes. The first pass opens with the ranks' ``prior_blocks``
    (one after another, no delay; ``app/linear_method/darlin.h:76-82``). With
    ``save_every = n`` and ``save_fn(iteration)`` the model is written after every
    n-th pass (``save_model_every_n_iter``, ``darlin.h:97-100``)."""
    cfg = ranks[0].cfg
    tau = cfg.tau if len(ranks) == 1 or all_reduce is not None else 0   # emulated ranks share a stream: no delay
    nb = len(ranks[0].blocks)
    history = []
    ts = 0
    reset_kkt = False
    n_ex = num_examples or sum(r.n_rows for r in ranks)
    if len(ranks) == 1:
        ranks[0]._pass_arrays()                    # host work that is not part of a pass
    for it in range(cfg.max_pass):
        order = list(range(nb))
        if cfg.random_block_order:
            np.random.default_rng(1000 + it).shuffle(order)
        if reset_kkt:
            for r in ranks:
                r.reset_kkt_filter()
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        ev[0].record()
        if len(ranks) == 1:
            # one rank per GPU: the whole pass is one persistent kernel (the prior blocks, one after
            # another, form a pass of their own with no delay)
            r = ranks[0]
            if it == 0 and r.prior_blocks:
                r.run_pass(r.prior_blocks, ts, 0)
                ts += len(r.prior_blocks)
            r.run_pass(order, ts, tau)
        else:
            # ranks emulated on one GPU: their kernels run one after another, block by block
            if it == 0 and ranks[0].prior_blocks:
                for blk in ranks[0].prior_blocks:
                    for r in ranks:
                        r.grad(blk, ts)
                    for r in ranks:
                        r.update(blk, ts)
                    for r in ranks:
                        r.dual(blk, ts)
                    ts += 1
            for i in range(len(order) + tau):
                if i < len(order):
                    for r in ranks:
                        r.grad(order[i], ts + i)
                j = i - tau
                if j >= 0:
                    for r in ranks:
                        r.update(order[j], ts + j)
                    for r in ranks:
                        r.dual(order[j], ts + j)
        ts += len(order)
        ev[1].record()
        loss = l1 = nnz = act = vio = 0.0
        for r in ranks:
            a = r.evaluate()
            loss += a[0]; l1 += a[1]; nnz += a[2]; act += a[3]; vio = max(vio, a[4])
            r.check_status()
        if all_reduce is not None:
            loss, l1, nnz, act = all_reduce([loss, l1, nnz, act], "sum")
            vio = all_reduce([vio], "max")[0]
        obj = loss + l1
        rel = (history[-1]["objective"] - obj) / history[-1]["objective"] if history else 1.0
        history.append(dict(iter=it, objective=obj, relative=rel, nnz_w=int(nnz), violation=vio, active=int(act),
                            device_ms=ev[0].elapsed_time(ev[1])))      # the pass on the device (evaluate() has synchronised)
        if verbose:
            print(f" {it:5d} | {obj:.5e}  {rel:.3e}  {int(nnz):8d} | {vio:.3e}  {int(act):9d}")
        thr = vio / max(1, n_ex) * cfg.kkt_ratio
        for r in ranks:
            r.kkt_threshold = thr
        if save_every > 0 and save_fn is not None and (it + 1) % save_every == 0:
            save_fn(it)
        if 0 < rel <= cfg.epsilon:
            if reset_kkt:
                break
            reset_kkt = True
        else:
            reset_kkt = False
    return history
