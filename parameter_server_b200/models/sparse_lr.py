"""Flagship model: sparse logistic regression trained through the device
parameter server (async SGD family: FTRL-proximal / AdaGrad / SGD).

One :class:`SparseLRWorker` per rank drives the per-minibatch pipeline

    H2D copy -> sort/unique/remap (K1) -> pull + margins + loss (F2)
             -> X^T g + scatter to owners (F1a) -> owner apply (F1b)

which is the worker/server loop of the reference's ``AsyncSGDWorker`` and
``AsyncSGDServer`` (``app/linear_method/async_sgd.h:42-310``) with the socket
round trips replaced by peer loads/stores. Minibatch ``t`` may start its pull
once every shard has applied round ``t - tau - 1`` (bounded delay).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..ops import _lib
from ..ops.localize import LocalBatch
from ..utils.idpack import PackedIds
from ..parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig
from ..parallel.fabric import Fabric


@dataclass
class SparseLRConfig:
    max_rows: int
    max_nnz: int
    tau: int = 0                       # bounded delay (minibatches)
    hash_seed: Optional[int] = 0       # hash raw ids to uint64 keys on the device; None: ids are keys
    key_bits: int = 64                 # sorted key bit range: int or (begin, end)
    hash_bits: int = 0                 # significant bits of device-hashed keys (0 = 64), placed in the top bits
    loss: str = "logit"
    real_values: bool = False
    pipeline: int = 3                  # minibatches in flight on the worker: copy | localise | pull+push
    auc: bool = False
    nvtx: bool = False                 # NVTX ranges around the stages of submit() for timeline profilers
    graph_localize: bool = True        # replay the localisation of a repeated call from a CUDA graph


class SparseLRWorker:
    def __init__(self, plane: DataPlane, cfg: SparseLRConfig):
        self.plane, self.cfg = plane, cfg
        dev = plane.device
        assert plane.cfg.ring >= cfg.tau + 2 or plane.S == 1 and plane.cfg.ring >= 1
        self.bufs: List[LocalBatch] = [
            LocalBatch(cfg.max_rows, cfg.max_nnz, plane.S, dev, real_values=cfg.real_values)
            for _ in range(max(1, cfg.pipeline))]
        self.step_no = 0
        self.loss_code = _lib.LOSS_LOGIT if cfg.loss == "logit" else _lib.LOSS_SQUARE_HINGE
        self.auc_hist = torch.zeros(2 * 4096, dtype=torch.int32, device=dev) if cfg.auc else None
        # streams: copy (H2D), prep (localise), main (pull/push), server (apply)
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.prep_stream = torch.cuda.Stream(device=dev)
        self.main_stream = torch.cuda.Stream(device=dev)
        self.server_stream = torch.cuda.Stream(device=dev)
        self._prep_done = [torch.cuda.Event() for _ in self.bufs]
        self._copy_done = [torch.cuda.Event() for _ in self.bufs]
        self._buf_free = [torch.cuda.Event() for _ in self.bufs]
        self._push_done = torch.cuda.Event()
        # one event per ring slot, recorded after the apply of that round
        self._applied_ev = [torch.cuda.Event() for _ in range(self.cfg.tau + 2)]
        self._staged = [None] * len(self.bufs)

    # ------------------------------------------------------------ pieces
    def prepare(self, ids: torch.Tensor, y: torch.Tensor, *, fixed_z: int = 0, row_ptr=None, vals=None,
                slot: Optional[int] = None, stream=None) -> LocalBatch:
        """Localise a minibatch whose tensors already live on the device."""
        slot = self.step_no % len(self.bufs) if slot is None else slot
        b = self.bufs[slot]
        b.localize(ids, y, self.plane.bounds, fixed_z=fixed_z, row_ptr=row_ptr, vals=vals,
                   hash_seed=self.cfg.hash_seed, key_bits=self.cfg.key_bits, hash_bits=self.cfg.hash_bits, stream=stream)
        return b

    def train_prepared(self, b: LocalBatch, stream=None, server_stream=None):
        """Pull + margins, push, apply for a localised batch (round = step number)."""
        t = self.step_no
        need = max(0, t - self.cfg.tau)
        if self.plane.cfg.pull_cap:
            self.plane.pull_exchange(b, t, need_applied=need, loss=self.loss_code, auc_hist=self.auc_hist, stream=stream)
            self.plane.push(b, t, send_keys=False, stream=stream)
        else:
            if self.plane.cfg.key_cache:
                self.plane.key_signature(b, stream=stream)
            self.plane.pull_margin(b, need_applied=need, loss=self.loss_code, auc_hist=self.auc_hist, stream=stream)
            self.plane.push(b, t, stream=stream)
        self.plane.apply(t, stream=server_stream if server_stream is not None else stream)
        self.step_no += 1

    # ------------------------------------------------------------ simple synchronous step
    def step(self, ids: torch.Tensor, y: torch.Tensor, *, fixed_z: int = 0, row_ptr=None, vals=None):
        """One minibatch on the current stream (device tensors)."""
        b = self.prepare(ids, y, fixed_z=fixed_z, row_ptr=row_ptr, vals=vals)
        self.train_prepared(b)
        return b

    # ------------------------------------------------------------ pipelined public API
    COPY_PIECE_BYTES = 3 << 19          # 1.5 MB

    def submit(self, ids: torch.Tensor, y: torch.Tensor, *, fixed_z: int = 0, row_ptr=None, vals=None):
        """Enqueue one minibatch. ``ids``/``y`` (and ``vals``/``row_ptr``) may be
        pinned host tensors -- they are copied on the copy stream -- or device
        tensors. Three minibatches are in flight: the copy of t+2, the localisation
        of t+1 (prep stream) and the pull/push/apply of t (main and server streams)."""
        k = self.step_no % len(self.bufs)
        b = self.bufs[k]
        dev = self.plane.device
        cur = torch.cuda.current_stream(dev)
        mark = torch.cuda.nvtx.range_push if self.cfg.nvtx else (lambda name: None)
        done = torch.cuda.nvtx.range_pop if self.cfg.nvtx else (lambda: None)
        mark(f"submit {self.step_no}: copy")
        # stage 1, copy stream: host -> device into this buffer's staging area (reusable once the
        # localise that last read it has finished)
        self.copy_stream.wait_stream(cur)
        self.copy_stream.wait_event(self._prep_done[k])
        self.copy_stream.wait_event(self._buf_free[k])   # labels / row offsets / values are read until the push
        with torch.cuda.stream(self.copy_stream):
            def to_dev(t, name):
                if isinstance(t, PackedIds):                # ids as a bit stream: copy the words, keep width and count
                    return t if t.is_cuda else PackedIds(to_dev(t.words, name), t.bits, t.n)
                if t is None or t.is_cuda:
                    return t
                st = self._staged[k] = self._staged[k] or {}
                d = st.get(name)
                if d is None or d.numel() < t.numel() or d.dtype != t.dtype:
                    d = st[name] = torch.empty(t.numel(), dtype=t.dtype, device=dev)
                v = d[:t.numel()]
                # A large input goes over in pieces: the launch commands of the kernels that run meanwhile are
                # fetched over the same PCIe link, and between two pieces they get through (one 50 MB copy
                # delayed a concurrent localisation by 30 %, 1.5 MB pieces by 7 %).
                step = max(1, self.COPY_PIECE_BYTES // t.element_size())
                if t.numel() > 2 * step:
                    t1, v1 = t.reshape(-1), v.reshape(-1)
                    for o in range(0, t1.numel(), step):
                        v1[o:o + step].copy_(t1[o:o + step], non_blocking=True)
                else:
                    v.copy_(t, non_blocking=True)
                return v
            ids_d, y_d = to_dev(ids, "ids"), to_dev(y, "y")
            vals_d, rp_d = to_dev(vals, "vals"), to_dev(row_ptr, "row_ptr")
            self._copy_done[k].record(self.copy_stream)
        done()
        mark("localise")
        # stage 2, prep stream: sort + unique + remap (the buffer is free once its push has read it)
        self.prep_stream.wait_event(self._copy_done[k])
        self.prep_stream.wait_event(self._buf_free[k])
        loc = b.localize_replayed if self.cfg.graph_localize else b.localize
        with torch.cuda.stream(self.prep_stream):
            loc(ids_d, y_d, self.plane.bounds, fixed_z=fixed_z, row_ptr=rp_d, vals=vals_d,
                hash_seed=self.cfg.hash_seed, key_bits=self.cfg.key_bits, hash_bits=self.cfg.hash_bits,
                stream=self.prep_stream)
            self._prep_done[k].record(self.prep_stream)
        self.main_stream.wait_event(self._prep_done[k])
        done()
        mark("pull+push+apply")
        t = self.step_no
        need = max(0, t - self.cfg.tau)
        if need > 0:
            # The pull of round t needs this rank's apply of round need-1. Waiting for it on the
            # host side of the stream (instead of spinning in the pull kernel) matters: a resident,
            # spinning pull kernel can leave no room on the SMs for the apply kernel it waits for.
            self.main_stream.wait_event(self._applied_ev[(need - 1) % len(self._applied_ev)])
        if self.plane.cfg.pull_cap:
            # two-sided exchange: bulk traffic only, and the push of this round is values-only
            self.plane.pull_exchange(b, t, need_applied=need, loss=self.loss_code, auc_hist=self.auc_hist,
                                     stream=self.main_stream)
            self.plane.push(b, t, send_keys=False, stream=self.main_stream)
        else:
            if self.plane.cfg.key_cache:
                self.plane.key_signature(b, stream=self.main_stream)
            self.plane.pull_margin(b, need_applied=need, loss=self.loss_code, auc_hist=self.auc_hist,
                                   stream=self.main_stream)
            self.plane.push(b, t, stream=self.main_stream)
        self._buf_free[k].record(self.main_stream)
        self._push_done.record(self.main_stream)
        self.server_stream.wait_event(self._push_done)
        self.plane.apply(t, stream=self.server_stream)
        self._applied_ev[t % len(self._applied_ev)].record(self.server_stream)
        done()
        self.step_no += 1
        return b

    def wait(self):
        """Make the current stream wait for everything submitted so far."""
        cur = torch.cuda.current_stream(self.plane.device)
        cur.wait_stream(self.main_stream)
        cur.wait_stream(self.server_stream)
        cur.wait_stream(self.prep_stream)
        cur.wait_stream(self.copy_stream)

    def read_progress(self, reset: bool = True):
        """Device -> host read of the progress counters: dict with the summed
        loss, accuracy count and examples seen since the last reset (worker side)
        and nnz delta / sum w^2 / sum dw^2 / updates (server side)."""
        self.wait()
        p = self.plane
        both = torch.cat([p.pull_stats, p.push_stats]).cpu()
        if reset:
            p.pull_stats.zero_()
            p.push_stats.zero_()
        loss, correct, rows, _, d_nnz, w2, dw2, n_upd = both.tolist()
        return {"loss_sum": loss, "n_correct": correct, "n_examples": rows, "d_nnz": d_nnz,
                "weight_sum": w2, "delta_sum": dw2, "n_updates": n_upd}


def make_single_gpu(table_capacity: int, inbox_cap: int, opt: OptimizerConfig, cfg: SparseLRConfig,
                    device=None, quant: str = "none", ordered_slots: bool = False, pull_cap: int = 0) -> SparseLRWorker:
    """Convenience: one GPU hosting one shard and one worker."""
    ring = cfg.tau + 2
    pc = PlaneConfig(table_capacity=table_capacity, inbox_cap=inbox_cap, ring=ring, quant=quant,
                     ordered_slots=ordered_slots, pull_cap=pull_cap)
    from ..parallel.dataplane import heap_layout
    fab = Fabric.single(heap_layout(pc, 1).total(), device)
    return SparseLRWorker(DataPlane(fab, pc, opt), cfg)
