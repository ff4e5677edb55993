"""NCCL all-to-all-v push/pull: the baseline the fused kernels are measured against.

Same minibatch pipeline and the same local kernels (sort/localise, table gather,
margins, X^T g, optimiser), but every byte that crosses GPUs goes through
``torch.distributed.all_to_all_single`` with split sizes, as a conventional
implementation would do it:

    counts exchange (the split sizes have to be on the host)
    pull : keys -> owners | local table gather (slots remembered) | values -> workers
    push : values -> owners (keys and slots are reused from the pull) | local apply

To keep the comparison fair the baseline gets what the fused path has: the split
sizes of minibatch t+1 are exchanged and copied to the host while minibatch t
runs (``exchange_counts`` / ``step``), so no step waits for a device-to-host
copy of its own; the owner remembers the slots it found during the pull and the
apply reuses them; and the driver overlaps the localisation of the next
minibatch on another stream.

This path is a baseline, not the product.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import ApplyParams, PullParams, PushParams, check, ptr, stream_ptr
from .dataplane import DataPlane


class NcclPushPull:
    def __init__(self, plane: DataPlane, max_unique: int, group=None):
        self.plane, self.group = plane, group
        self.S, self.rank = plane.S, plane.rank
        dev = plane.device
        self.dev = dev
        cap = max_unique * 2 + 1024
        self.cap = cap
        i32, i64, f32 = torch.int32, torch.int64, torch.float32
        self.send_counts = torch.zeros(self.S, dtype=i64, device=dev)
        self.recv_counts = torch.zeros(self.S, dtype=i64, device=dev)
        self.rkeys = torch.empty(cap, dtype=i64, device=dev)      # keys received as an owner
        self.rvals = torch.empty(cap, dtype=f32, device=dev)      # weights gathered for the requesters
        self.rgrad = torch.empty(cap, dtype=f32, device=dev)      # gradients received as an owner
        self.stage = torch.empty(max_unique, dtype=f32, device=dev)
        self.stage_keys = torch.empty(max_unique, dtype=i64, device=dev)
        self.counts32 = torch.zeros(self.S, dtype=i32, device=dev)
        self.ready = torch.full((self.S,), 0x7FFFFFF0, dtype=i32, device=dev)
        self.dummy = torch.zeros(4 * self.S + 8, dtype=i32, device=dev)
        self.one_off = torch.zeros(2, dtype=i32, device=dev)
        self.n_recv = torch.zeros(1, dtype=i32, device=dev)
        self.slot_cache = torch.zeros(cap, dtype=i32, device=dev)
        self.collectives = 0
        # split sizes of two minibatches in flight: device tensors, pinned host copies, copy-done events
        self._sc_dev = [torch.zeros(self.S, dtype=i64, device=dev) for _ in range(2)]
        self._rc_dev = [torch.zeros(self.S, dtype=i64, device=dev) for _ in range(2)]
        self._sc_host = [torch.zeros(self.S, dtype=i64).pin_memory() for _ in range(2)]
        self._rc_host = [torch.zeros(self.S, dtype=i64).pin_memory() for _ in range(2)]
        self._counts_ev = [torch.cuda.Event() for _ in range(2)]

    def exchange_counts(self, b, k: int):
        """Exchange the split sizes of localised batch ``b`` (slot ``k`` of two) on the current stream and
        start their copy to the host; ``step(..., counts_slot=k)`` picks them up later."""
        self._sc_dev[k].copy_((b.own_off[1:] - b.own_off[:-1]).to(torch.int64))
        dist.all_to_all_single(self._rc_dev[k], self._sc_dev[k], group=self.group)
        self._sc_host[k].copy_(self._sc_dev[k], non_blocking=True)
        self._rc_host[k].copy_(self._rc_dev[k], non_blocking=True)
        self._counts_ev[k].record()
        self.collectives += 1

    def step(self, b, t: int, loss: int = 0, counts_slot: int = -1):
        """One minibatch (already localised into ``b``) through NCCL push/pull. With ``counts_slot`` the
        split sizes come from an earlier ``exchange_counts``; otherwise they are exchanged here."""
        p, S, L = self.plane, self.S, _lib.lib()
        sp = stream_ptr()
        # ---- split sizes (the all-to-all-v needs them on the host)
        if counts_slot >= 0:
            self._counts_ev[counts_slot].synchronize()      # recorded a whole step ago: normally no wait at all
            sc = self._sc_host[counts_slot].tolist()
            rc = self._rc_host[counts_slot].tolist()
            self.recv_counts.copy_(self._rc_dev[counts_slot])
        else:
            self.send_counts.copy_((b.own_off[1:] - b.own_off[:-1]).to(torch.int64))
            dist.all_to_all_single(self.recv_counts, self.send_counts, group=self.group)
            sc = self.send_counts.tolist()
            rc = self.recv_counts.tolist()
        U, R = sum(sc), sum(rc)
        assert R <= self.cap
        # ---- pull: keys to the owners
        dist.all_to_all_single(self.rkeys[:R], b.ukeys[:U], rc, sc, group=self.group)
        # owner: gather from the local table
        self.n_recv.fill_(R)
        self.one_off.copy_(torch.tensor([0, R], dtype=torch.int32))
        g = PullParams()
        g.S, g.insert = 1, 1                     # absent keys are inserted on first touch, as in the fused pull
        g.slot_local = ptr(self.slot_cache)      # ... and the slots are remembered for the apply
        g.table[0], g.mask[0] = p.table_ptr(), p.cfg.table_capacity - 1
        g.key_begin[0], g.slot_mult[0] = p.bounds_host[self.rank], p.slot_mult[self.rank]
        g.applied[0], g.need_applied = p._ctrl(self.rank, 0), 0
        g.ukeys, g.n_unique, g.own_off = ptr(self.rkeys), ptr(self.n_recv), ptr(self.one_off)
        g.w_local, g.n_rows = ptr(self.rvals), 0
        g.stats, g.bar, g.status = ptr(p.pull_stats), p._bar(0), ptr(p.status)
        check(L.psb_pull_margin(C.byref(g), sp), "gather")
        # values back to the workers
        dist.all_to_all_single(b.w_local[:U], self.rvals[:R], sc, rc, group=self.group)
        # ---- margins + loss (gather skipped)
        m = PullParams()
        m.S, m.insert = S, 2
        m.ukeys, m.n_unique, m.own_off = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off)
        m.w_local, m.grad_zero = ptr(b.w_local), ptr(b.grad)
        m.row_ptr, m.n_rows, m.fixed_z = ptr(b.row_ptr), b.n_rows, b.fixed_z
        m.csr_col, m.csr_val, m.y, m.loss = ptr(b.csr_col), ptr(b.csr_val), ptr(b.y), loss
        m.gcoef, m.margin = ptr(b.gcoef), ptr(b.margin)
        m.stats, m.bar, m.status = ptr(p.pull_stats), p._bar(0), ptr(p.status)
        check(L.psb_pull_margin(C.byref(m), sp), "margins")
        # ---- X^T g into a contiguous staging buffer (same kernel, local destinations)
        q = PushParams()
        q.S, q.ts1, q.inbox_cap, q.quant, q.send_keys = S, t + 1, self.stage.numel(), 0, 0
        off = 0
        for s in range(S):
            q.inbox_keys[s] = self.stage_keys.data_ptr() + off * 8
            q.inbox_vals[s] = self.stage.data_ptr() + off * 4
            q.ready[s] = self.dummy.data_ptr() + 4 * s
            q.count[s] = self.dummy.data_ptr() + 4 * (S + s)
            q.applied[s] = self.dummy.data_ptr()
            off += sc[s]
        q.need_applied = 0
        q.ukeys, q.n_unique, q.own_off = ptr(b.ukeys), ptr(b.n_unique), ptr(b.own_off)
        q.nnz, q.csc_row, q.csc_val = b.nnz, ptr(b.csc_row), ptr(b.csc_val)
        q.flagbits, q.wordbase, q.gcoef, q.grad = ptr(b.flagbits), ptr(b.wordbase), ptr(b.gcoef), ptr(b.grad)
        q.bar, q.done, q.status = p._bar(1), p._done(1), ptr(p.status)
        check(L.psb_push(C.byref(q), sp), "grad")
        # ---- push: values to the owners (the owners still hold the keys of this round)
        dist.all_to_all_single(self.rgrad[:R], self.stage[:U], rc, sc, group=self.group)
        # ---- owner: duplicate-key reduce + optimiser on the received segments
        self.counts32.copy_(self.recv_counts.to(torch.int32))
        a = ApplyParams()
        a.S, a.ts1, a.inbox_cap, a.quant = S, t + 1, self.cap, 0
        a.table, a.mask = p.table_ptr(), p.cfg.table_capacity - 1
        a.key_begin, a.slot_mult = p.bounds_host[self.rank], p.slot_mult[self.rank]
        off = 0
        for r in range(S):
            a.inbox_keys[r] = self.rkeys.data_ptr() + off * 8
            a.inbox_vals[r] = self.rgrad.data_ptr() + off * 4
            a.ready[r] = self.ready.data_ptr() + 4 * r
            a.count[r] = self.counts32.data_ptr() + 4 * r
            a.alive[r], a.cached[r] = 1, 1       # slots found by the gather above
            a.slot_cache[r] = self.slot_cache.data_ptr() + off * 4
            off += rc[r]
        a.opt = p.opt.to_c()
        a.stats, a.applied = ptr(p.push_stats), p._ctrl(self.rank, 0)
        a.bar, a.done, a.status = p._bar(2), p._done(2), ptr(p.status)
        check(L.psb_apply(C.byref(a), sp), "apply")
        self.collectives += 3 if counts_slot >= 0 else 4


class NcclKV:
    """Push and pull of sorted unique keys with ``k``-wide values the conventional way, for the KV
    microbenchmark: all-to-all-v of keys and values through NCCL, then the owner's look-up and merge
    with the library's own table kernels (``k_apply`` over the received segments; ``k_pull_margin`` as a
    local gather that remembers the slots). It works on the local shard of ``plane`` (table, key range
    and slot map are the plane's), so both arms of the benchmark hit the same table.

    The split sizes are computed once per key list on the host (``set_keys``): the benchmark repeats
    its key list, and a real implementation would have to exchange them every round."""

    def __init__(self, plane: DataPlane, max_keys: int, group=None):
        self.plane, self.group = plane, group
        self.S, self.rank, self.k = plane.S, plane.rank, plane.width
        dev = self.dev = plane.device
        cap = self.cap = max_keys * 2 + 1024
        i32, i64, f32 = torch.int32, torch.int64, torch.float32
        self.rkeys = torch.empty(cap, dtype=i64, device=dev)
        self.rvals = torch.empty(cap * self.k, dtype=f32, device=dev)
        self.rw = torch.empty(cap, dtype=f32, device=dev)
        self.slot_cache = torch.zeros(cap, dtype=i32, device=dev)
        self.counts32 = torch.zeros(self.S, dtype=i32, device=dev)
        self.ready = torch.full((self.S,), 0x7FFFFFF0, dtype=i32, device=dev)
        self.dummy = torch.zeros(64, dtype=i32, device=dev)
        self.one_off = torch.zeros(2, dtype=i32, device=dev)
        self.n_recv = torch.zeros(1, dtype=i32, device=dev)
        self.t = 0

    def set_keys(self, keys_u64):
        """Split sizes of a sorted unique uint64 key list (NumPy) by the plane's key ranges."""
        import numpy as np
        inner = np.array(self.plane.bounds_host[1:-1], dtype=np.uint64)
        cuts = np.concatenate([[0], np.searchsorted(keys_u64, inner), [len(keys_u64)]])
        self.sc = np.diff(cuts).astype(np.int64).tolist()
        cin = torch.zeros(self.S, dtype=torch.int64, device=self.dev)
        if self.S > 1:
            dist.all_to_all_single(cin, torch.tensor(self.sc, dtype=torch.int64, device=self.dev), group=self.group)
        else:
            cin[0] = self.sc[0]
        self.rc = cin.tolist()
        self.R = sum(self.rc)
        assert self.R <= self.cap
        self.counts32.copy_(cin.to(torch.int32))
        self.n_recv.fill_(self.R)
        self.one_off.copy_(torch.tensor([0, self.R], dtype=torch.int32))

    def _a2a(self, out, inp, osz, isz, width=1):
        out, inp = out.reshape(-1), inp.reshape(-1)
        if self.S == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out, inp, [n * width for n in osz], [n * width for n in isz], group=self.group)

    def push(self, keys: torch.Tensor, vals: torch.Tensor):
        p, S, k, L = self.plane, self.S, self.k, _lib.lib()
        R = self.R
        self._a2a(self.rkeys[:R], keys, self.rc, self.sc)
        self._a2a(self.rvals[:R * k], vals.reshape(-1), self.rc, self.sc, k)
        a = ApplyParams()
        a.S, a.ts1, a.inbox_cap, a.quant = S, self.t + 1, self.cap, 0
        a.table, a.mask = p.table_ptr(), p.cfg.table_capacity - 1
        a.key_begin, a.slot_mult = p.bounds_host[self.rank], p.slot_mult[self.rank]
        off = 0
        for r in range(S):
            a.inbox_keys[r] = self.rkeys.data_ptr() + off * 8
            a.inbox_vals[r] = self.rvals.data_ptr() + off * k * 4
            a.ready[r] = self.ready.data_ptr() + 4 * r
            a.count[r] = self.counts32.data_ptr() + 4 * r
            a.alive[r], a.cached[r] = 1, 0
            a.slot_cache[r] = self.slot_cache.data_ptr() + off * 4
            off += self.rc[r]
        a.opt = p.opt.to_c()
        a.stats, a.applied = ptr(p.push_stats), self.dummy.data_ptr() + 128
        a.bar, a.done, a.status = p._bar(2), p._done(2), ptr(p.status)
        a.width, a.wide_vals = k, p.wide_vals_ptr(0)
        check(L.psb_apply(C.byref(a), stream_ptr()), "apply")
        self.t += 1

    def pull(self, keys: torch.Tensor, out: torch.Tensor):
        p, k, L = self.plane, self.k, _lib.lib()
        R = self.R
        self._a2a(self.rkeys[:R], keys, self.rc, self.sc)
        g = PullParams()
        g.S, g.insert = 1, 1
        g.slot_local = ptr(self.slot_cache)
        g.table[0], g.mask[0] = p.table_ptr(), p.cfg.table_capacity - 1
        g.key_begin[0], g.slot_mult[0] = p.bounds_host[self.rank], p.slot_mult[self.rank]
        g.applied[0], g.need_applied = self.dummy.data_ptr() + 128, 0
        g.ukeys, g.n_unique, g.own_off = ptr(self.rkeys), ptr(self.n_recv), ptr(self.one_off)
        g.w_local, g.n_rows = ptr(self.rw), 0
        g.stats, g.bar, g.status = ptr(p.pull_stats), p._bar(0), ptr(p.status)
        check(L.psb_pull_margin(C.byref(g), stream_ptr()), "gather")
        if k == 1:
            self._a2a(out, self.rw[:R], self.sc, self.rc)
        else:
            wide = p.fabric.view(p.layout["wide_vals"], (p.cfg.table_capacity, k), torch.float32)
            torch.index_select(wide, 0, self.slot_cache[:R].long(), out=self.rvals[:R * k].view(R, k))
            self._a2a(out.reshape(-1), self.rvals[:R * k], self.sc, self.rc, k)
