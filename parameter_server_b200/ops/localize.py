"""Minibatch localisation on the GPU: unique keys + CSC/CSR remap (kernels K1/K2).

:class:`LocalBatch` owns every per-minibatch device buffer of a worker, sized
once for the largest minibatch, so a training step allocates nothing.

Two device paths produce the same outputs. ``bucket`` groups the nonzeros by
key without a full sort (frequent keys by counting, the rest per key-range
bucket in shared memory); it assumes keys that are spread evenly over the key
space (hashed keys) and raises a device flag otherwise. ``sort`` is the radix
sort + head-flag scan. ``auto`` (the default) enqueues ``bucket`` and, behind
it, the ``sort`` kernels gated on that flag, so the result is right for any
input and nothing waits for the host.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr
from ..utils.idpack import PackedIds


def sort_pairs(keys: torch.Tensor, payload: Optional[torch.Tensor] = None, begin_bit: int = 0,
               end_bit: int = 64, stream=None):
    """Sort int64-viewed uint64 ``keys`` (and a uint32 payload, default = index).
    Returns ``(sorted_keys, sorted_payload)`` as new tensors."""
    n = keys.numel()
    dev = keys.device
    ka = keys.clone()
    kb = torch.empty_like(ka)
    va = payload.clone() if payload is not None else torch.empty(n, dtype=torch.int32, device=dev)
    vb = torch.empty_like(va)
    L = _lib.lib()
    scratch = torch.empty(L.psb_sort_scratch_bytes(n, begin_bit, end_bit), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    where = torch.zeros(1, dtype=torch.int32, device=dev)
    check(L.psb_sort_pairs(ptr(ka), 0, 0, ptr(ka), ptr(va), int(payload is not None), ptr(kb), ptr(vb),
                           n, begin_bit, end_bit, ptr(scratch), ptr(status), ptr(where), 0, stream_ptr(stream)), "sort",
          kernels=3 + (end_bit - begin_bit + 7) // 8)
    _lib.check_status(status, "radix sort")
    in_b = int(where.item()) == 1
    return (kb, vb) if in_b else (ka, va)


class LocalBatch:
    """Device buffers of one in-flight minibatch of a worker."""

    BUCKET_MIN_NNZ = 4096      # below this the sort path is as fast and has fewer launches

    def __init__(self, max_rows: int, max_nnz: int, n_shards: int, device, real_values: bool = False):
        dev = device
        i32, i64, f32 = torch.int32, torch.int64, torch.float32
        self.device, self.max_rows, self.max_nnz, self.S = dev, max_rows, max_nnz, n_shards
        L = _lib.lib()
        self.keys_a = torch.empty(max_nnz, dtype=i64, device=dev)
        self.keys_b = torch.empty(max_nnz, dtype=i64, device=dev)
        self.pos_a = torch.empty(max_nnz, dtype=i32, device=dev)
        self.pos_b = torch.empty(max_nnz, dtype=i32, device=dev)
        self.csc_row_buf = torch.empty(max_nnz, dtype=i32, device=dev)
        self.where = torch.zeros(1, dtype=i32, device=dev)   # which ping-pong buffer holds the sorted pairs
        nb = max(L.psb_sort_scratch_bytes(max_nnz, 0, 64), L.psb_localize_scratch_bytes(max_nnz))
        self.scratch = torch.empty(nb, dtype=torch.uint8, device=dev)
        self.bucket_scratch = torch.empty(L.psb_bucket_localize_scratch_bytes(max_nnz), dtype=torch.uint8, device=dev)
        self.gate = torch.zeros(1, dtype=i32, device=dev)    # 1 = the bucket path gave up on this minibatch
        self.status = torch.zeros(1, dtype=i32, device=dev)
        self.ukeys = torch.empty(max_nnz, dtype=i64, device=dev)
        self.seg_off = torch.empty(max_nnz + 1, dtype=i32, device=dev)
        self.csr_col = torch.empty(max_nnz, dtype=i32, device=dev)
        self.flagbits = torch.empty((max_nnz + 31) // 32, dtype=i32, device=dev)
        self.wordbase = torch.empty((max_nnz + 31) // 32, dtype=i32, device=dev)
        self.n_unique = torch.zeros(1, dtype=i32, device=dev)
        self.own_off = torch.zeros(n_shards + 1, dtype=i32, device=dev)
        self.w_local = torch.empty(max_nnz, dtype=f32, device=dev)
        self.grad = torch.zeros(max_nnz, dtype=f32, device=dev)
        self.slot_local = None
        self.key_hit = torch.zeros(1, dtype=i32, device=dev)     # key-caching filter: 1 = same list as last time
        self.key_sig = torch.zeros(4, dtype=i32, device=dev)
        self.gcoef = torch.empty(max_rows, dtype=f32, device=dev)
        self.margin = torch.empty(max_rows, dtype=f32, device=dev)
        self.csc_val_buf = torch.empty(max_nnz, dtype=f32, device=dev) if real_values else None
        # set per batch
        self.n_rows = 0
        self.nnz = 0
        self.fixed_z = 0
        self.row_ptr = None
        self.csr_val = None
        self.csc_val = None
        self.csc_row = None
        self.y = None

    def localize(self, ids: torch.Tensor, y: Optional[torch.Tensor], bounds: torch.Tensor, *,
                 fixed_z: int = 0, row_ptr: Optional[torch.Tensor] = None,
                 vals: Optional[torch.Tensor] = None, hash_seed: Optional[int] = None,
                 key_bits=64, hash_bits: int = 0, packed: Optional[bool] = None, method: str = "auto",
                 stream=None):
        """Sort + unique + remap one minibatch.

        ``ids``: flat per-nonzero feature ids. ``int32`` (raw ids, hashed to uint64
        keys on the device when ``hash_seed`` is given) or ``int64`` (already
        uint64 keys viewed as int64, or raw ids to hash when ``hash_seed`` is given).
        Rows are given by ``row_ptr`` (CSR offsets, int32) or a fixed ``fixed_z``
        nonzeros per row. ``hash_bits`` (0 = 64) is the number of significant bits
        of the hashed keys, which sit in the top bits; ``key_bits`` is the sorted
        bit range, an int (``[0, key_bits)``) or a ``(begin, end)`` pair. Digit
        positions that turn out constant across the batch are skipped anyway.
        ``packed``: None = pack (key, position) into one word whenever possible,
        False = never, True = require it. ``method``: ``auto`` | ``bucket`` |
        ``sort`` (see the module docstring); inside a key's CSC segment the
        bucket path lists the rows in no particular order, the sort path by
        position.
        """
        L = _lib.lib()
        if isinstance(ids, PackedIds):
            # a bit stream from the loader: unpack to 32-bit ids first (part of the same launch sequence,
            # so a replayed graph contains it)
            n = ids.n
            assert n <= self.max_nnz and ids.words.is_cuda and hash_seed is not None
            if self.__dict__.get("_ids32") is None:
                self._ids32 = torch.empty(self.max_nnz, dtype=torch.int32, device=self.device)
            check(L.psb_unpack_ids(ptr(ids.words), ids.bits, n, ptr(self._ids32), stream_ptr(stream)), "unpack ids")
            ids = self._ids32[:n]
        n = ids.numel()
        assert n <= self.max_nnz
        self.nnz = n
        if row_ptr is not None:
            self.n_rows = row_ptr.numel() - 1
            self.fixed_z = 0
        else:
            assert fixed_z > 0 and n % fixed_z == 0
            self.n_rows = n // fixed_z
            self.fixed_z = fixed_z
        assert self.n_rows <= self.max_rows
        self.row_ptr, self.csr_val, self.y = row_ptr, vals, y
        sp = stream_ptr(stream)
        if hash_seed is None:
            assert ids.dtype == torch.int64
            in_kind, seed = 0, 0
        else:
            in_kind, seed = (1 if ids.dtype == torch.int32 else 2), hash_seed | (hash_bits << 56)
        lo_bit, hi_bit = key_bits if isinstance(key_bits, tuple) else (0, key_bits)
        # Packed mode: narrow hashed keys leave their low bits zero; when every element index fits there,
        # (key, position) travels as one 64-bit word and the sort needs no payload array.
        pack = 0
        if packed is not False and hash_seed is not None and 0 < hash_bits < 64 and n > 0:
            free = min(64 - hash_bits, 32)
            if (n - 1) >> free == 0:
                pack = free
                lo_bit = max(lo_bit, 64 - hash_bits)
        assert pack or not packed, "packed mode needs hashed keys with (64 - hash_bits) bits for the positions"
        self.pack_bits = pack
        self.csc_val = self.csc_val_buf if vals is not None else None
        if vals is not None:
            assert self.csc_val_buf is not None
        self.csc_row = self.csc_row_buf
        assert method in ("auto", "bucket", "sort")
        # the bucket path takes its buckets from the top key bits: only for keys sorted up to bit 64
        use_bucket = method != "sort" and hi_bit == 64 and n >= self.BUCKET_MIN_NNZ
        gate = 0
        if use_bucket:
            low_zero = (64 - hash_bits) if (hash_seed is not None and 0 < hash_bits < 64) else 0
            check(L.psb_bucket_localize(ptr(ids), in_kind, seed, n, low_zero, ptr(row_ptr), self.n_rows, self.fixed_z,
                                        ptr(vals), ptr(bounds), self.S, ptr(self.keys_a), ptr(self.pos_a),
                                        ptr(self.keys_b), ptr(self.ukeys), ptr(self.seg_off), ptr(self.csr_col),
                                        ptr(self.csc_row_buf), ptr(self.csc_val), ptr(self.flagbits),
                                        ptr(self.wordbase), ptr(self.n_unique), ptr(self.own_off),
                                        ptr(self.bucket_scratch), ptr(self.status), ptr(self.gate), sp),
                  "bucket localize", kernels=10)
            if method == "bucket":
                return self
            gate = ptr(self.gate)
        # sort-based path; behind the bucket path its kernels run only if that one raised the gate
        check(L.psb_sort_pairs_gated(ptr(ids), in_kind, seed, ptr(self.keys_a), 0 if pack else ptr(self.pos_a), 0,
                                     ptr(self.keys_b), 0 if pack else ptr(self.pos_b), n, lo_bit, hi_bit,
                                     ptr(self.scratch), ptr(self.status), ptr(self.where), pack, gate, sp), "sort",
              kernels=3 + (hi_bit - lo_bit + 7) // 8)
        check(L.psb_localize2_gated(ptr(self.keys_a), ptr(self.keys_b), ptr(self.pos_a), ptr(self.pos_b),
                                    ptr(self.where), ptr(self.csc_row_buf), n, ptr(row_ptr), self.n_rows,
                                    self.fixed_z, ptr(vals), ptr(bounds), self.S, ptr(self.ukeys), ptr(self.seg_off),
                                    ptr(self.csr_col), ptr(self.csc_val), ptr(self.flagbits), ptr(self.wordbase),
                                    ptr(self.n_unique), ptr(self.own_off), ptr(self.scratch), pack, gate, sp),
              "localize", kernels=4)
        return self

    MAX_GRAPHS = 16

    def localize_replayed(self, ids: torch.Tensor, y: Optional[torch.Tensor], bounds: torch.Tensor, *, stream,
                          row_ptr: Optional[torch.Tensor] = None, vals: Optional[torch.Tensor] = None, **kw):
        """:meth:`localize` on ``stream``, replayed from a CUDA graph once the same call (the same input
        tensors at the same addresses, the same arguments) comes a second time: a training loop that
        stages its minibatches in fixed buffers then pays one graph launch instead of some twenty
        kernel launches. That matters most while host-to-device copies keep PCIe busy, because the
        launch commands of plain kernels are fetched over the same link and queue behind the copies.
        Calls that never repeat (minibatches of varying size) run as plain launches."""
        def addr(t):
            if isinstance(t, PackedIds):
                return (t.words.data_ptr(), t.n, t.bits)
            return (0, 0) if t is None else (t.data_ptr(), t.numel())
        key = (addr(ids), None if isinstance(ids, PackedIds) else ids.dtype, addr(y), addr(bounds), addr(row_ptr), addr(vals),
               tuple(sorted((k, v) for k, v in kw.items())))
        graphs = self.__dict__.setdefault("_graphs", {})
        ent = graphs.get(key)
        if ent is None or ent == "seen" and sum(1 for v in graphs.values() if v != "seen") >= self.MAX_GRAPHS:
            if len(graphs) > 8 * self.MAX_GRAPHS:              # calls that never repeat: forget the marks
                for k in [k for k, v in graphs.items() if v == "seen"]:
                    del graphs[k]
            graphs[key] = "seen"
            with torch.cuda.stream(stream):
                return self.localize(ids, y, bounds, row_ptr=row_ptr, vals=vals, stream=stream, **kw)
        if ent == "seen":
            g = torch.cuda.CUDAGraph()
            before = _lib.LAUNCHES
            # thread_local: other threads of the process (loaders, node threads) may call the runtime meanwhile
            with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                self.localize(ids, y, bounds, row_ptr=row_ptr, vals=vals, stream=torch.cuda.current_stream(), **kw)
            state = {a: getattr(self, a) for a in ("nnz", "n_rows", "fixed_z", "row_ptr", "csr_val", "y", "pack_bits",
                                                   "csc_val", "csc_row")}
            ent = graphs[key] = (g, state, _lib.LAUNCHES - before, (ids, y, bounds, row_ptr, vals))
            _lib.LAUNCHES = before                             # the capture launched nothing
        g, state, kernels, _ = ent
        for a, v in state.items():
            setattr(self, a, v)
        with torch.cuda.stream(stream):
            g.replay()
        _lib.LAUNCHES += kernels
        return self

    def set_keys(self, ukeys_sorted: torch.Tensor, bounds, stream=None):
        """Use an already sorted unique key list (generic Push/Pull API path). ``bounds``
        is the device tensor of shard boundaries; the owner offsets are computed on
        the device, so nothing here waits for the host."""
        n = ukeys_sorted.numel()
        assert n <= self.max_nnz
        self.ukeys[:n].copy_(ukeys_sorted)
        self.n_unique.fill_(n)
        check(_lib.lib().psb_owner_offsets(ptr(self.ukeys), ptr(self.n_unique), ptr(bounds), self.S,
                                           ptr(self.own_off), stream_ptr(stream)), "owner offsets")
        self.n_rows = 0
        self.nnz = 0
        return self
