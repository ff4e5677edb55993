"""Preprocessing of the Darlin data on the device: tail-feature filter, the global
column space and the division into feature blocks.

What the reference does with three rounds of push/pull per feature group before
training starts (``learner/bcd.h:179-203,294-338``, ``learner/bcd.cc:78-116``):

* every worker counts how often each of its keys occurs, the counts are merged
  in a count-min sketch on the servers, and keys seen fewer than
  ``tail_feature_freq`` times are dropped (``FreqencyFilter``);
* the servers build the key set of every feature group (the union of the
  workers' remaining keys);
* every group's key range is cut into ``ceil(nnz per row * feature_block_ratio)``
  blocks; blocks of the ``prior_fea_group`` groups run first.

Here the counts go through the device count-min kernels, the sketches of the
ranks are merged with saturating adds, the union is a sort + unique of the
gathered key lists on the device, and every nonzero gets the index of its
column in the global column space (group-major, keys ascending inside a group).
The block kernels (``csrc/cuda/darlin.cu``) then work on column indices only.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops.localize import LocalBatch

_SIGN = -(1 << 63)


def _ordered(keys_i64: torch.Tensor) -> torch.Tensor:
    """uint64 keys viewed as int64 -> int64 values whose signed order is the keys' unsigned order."""
    return keys_i64 ^ _SIGN


def unique_with_counts(keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sorted unique keys (uint64 as int64), their counts and the index of every input key in the
    unique list, with the library's own sort + localise kernels."""
    n = keys.numel()
    dev = keys.device
    if n == 0:
        z = torch.zeros(0, dtype=torch.int64, device=dev)
        return z, torch.zeros(0, dtype=torch.int32, device=dev), torch.zeros(0, dtype=torch.int32, device=dev)
    b = LocalBatch(n, n, 1, dev)
    bounds = torch.tensor([0, -1], dtype=torch.int64, device=dev)
    b.localize(keys.contiguous(), None, bounds, fixed_z=1, hash_seed=None, method="sort")
    torch.cuda.synchronize(dev)
    U = int(b.n_unique.item())
    seg = b.seg_off[:U + 1]
    return b.ukeys[:U].clone(), (seg[1:] - seg[:-1]).clone(), b.csr_col[:n].clone()


def gather_union(local_unique: torch.Tensor, dist) -> torch.Tensor:
    """Sorted union of every rank's sorted unique key list."""
    if dist is None:
        return local_unique
    dev = local_unique.device
    world = dist.get_world_size()
    n = torch.tensor([local_unique.numel()], dtype=torch.int64, device=dev)
    sizes = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
    dist.all_gather(sizes, n)
    sizes = [int(s.item()) for s in sizes]
    cap = max(1, max(sizes))
    mine = torch.zeros(cap, dtype=torch.int64, device=dev)
    mine[:local_unique.numel()] = local_unique
    every = torch.zeros(world * cap, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(every, mine)
    parts = [every[r * cap:r * cap + sizes[r]] for r in range(world)]
    return unique_with_counts(torch.cat(parts))[0]


def tail_filter(unique_keys: torch.Tensor, counts: torch.Tensor, freq: int, sketch_cells: int, sketch_k: int,
                dist) -> torch.Tensor:
    """Mask over ``unique_keys``: the keys whose occurrences, summed over all ranks and estimated by a
    count-min sketch of ``sketch_cells`` saturating 8-bit cells and ``sketch_k`` probes, reach ``freq``."""
    from ..ops.filters import CountMin
    dev = unique_keys.device
    cm = CountMin(sketch_cells, sketch_k, dev)
    if unique_keys.numel():
        cm.insert(unique_keys, counts.clamp(max=255).to(torch.uint8))
    if dist is not None:
        world = dist.get_world_size()
        cells = cm.bytes().contiguous()
        every = torch.zeros(world * cells.numel(), dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(every, cells)
        merged = every.view(world, -1).to(torch.int32).sum(0).clamp(max=255).to(torch.uint8)
        cm.bytes().copy_(merged)
    if unique_keys.numel() == 0:
        return torch.zeros(0, dtype=torch.bool, device=dev)
    return cm.query(unique_keys) >= min(freq, 255)


@dataclass
class ColumnSpace:
    col_key: torch.Tensor                       # uint64 key (int64 view) of every global column
    groups: List[Tuple[int, int, int]]          # (group id, first column, one past the last)
    nnz_per_row: List[float]                    # per group, over all ranks (for the block division)
    dropped_nnz: int = 0

    @property
    def n_cols(self) -> int:
        return int(self.col_key.numel())


def build_columns(groups: Sequence[dict], n_rows: int, dev, *, dist=None, tail_freq: int = 0,
                  countmin_cells: int = 1 << 20, countmin_k: int = 2):
    """``groups``: one dict per feature group of this rank's rows, as the stream reader returns them
    (``id``, ``offset`` CSR row offsets, ``index`` uint64 keys, ``value`` or empty, ``binary``).
    Returns ``(col, row_ptr, vals, space)``: the column index of every remaining nonzero in CSR order
    over all groups (a row's nonzeros group by group), the new row offsets, the values (None when
    every group is binary) and the :class:`ColumnSpace`."""
    per_group = []
    space_keys, space_groups, nnz_per_row = [], [], []
    base = 0
    dropped = 0
    binary = all(g["binary"] for g in groups)
    total_rows = n_rows
    if dist is not None:
        t = torch.tensor([n_rows], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        total_rows = int(t.item())
    for g in sorted(groups, key=lambda d: d["id"]):
        keys = torch.from_numpy(np.ascontiguousarray(g["index"]).view(np.int64)).to(dev)
        off = torch.from_numpy(np.ascontiguousarray(g["offset"]).astype(np.int64)).to(dev)
        vals = None if binary else (torch.ones(keys.numel(), device=dev) if g["binary"]
                                    else torch.from_numpy(np.ascontiguousarray(g["value"])).to(dev))
        uk, cnt, inv = unique_with_counts(keys)
        keep_u = torch.ones(uk.numel(), dtype=torch.bool, device=dev)
        if tail_freq > 0:
            keep_u = tail_filter(uk, cnt, tail_freq, countmin_cells, countmin_k, dist)
        gk = gather_union(uk[keep_u], dist)                                    # the group's global key set
        keep_nz = keep_u[inv.long()] if keys.numel() else torch.zeros(0, dtype=torch.bool, device=dev)
        dropped += int((~keep_nz).sum().item())
        row_of = torch.repeat_interleave(torch.arange(off.numel() - 1, device=dev), off[1:] - off[:-1])
        kept_keys = keys[keep_nz]
        col = torch.searchsorted(_ordered(gk), _ordered(kept_keys)) + base if kept_keys.numel() else kept_keys
        per_group.append((row_of[keep_nz], col, None if vals is None else vals[keep_nz]))
        nnz_all = torch.tensor([float(kept_keys.numel())], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(nnz_all)
        space_keys.append(gk)
        space_groups.append((int(g["id"]), base, base + gk.numel()))
        nnz_per_row.append(float(nnz_all.item()) / max(1, total_rows))
        base += gk.numel()
    # rows back together: a row's nonzeros of group 0, then of group 1, ...
    rows = torch.cat([p[0] for p in per_group]) if per_group else torch.zeros(0, dtype=torch.int64, device=dev)
    cols = torch.cat([p[1] for p in per_group]) if per_group else rows
    order = torch.sort(rows, stable=True)[1]
    lens = torch.bincount(rows, minlength=n_rows)
    row_ptr = torch.zeros(n_rows + 1, dtype=torch.int64, device=dev)
    row_ptr[1:] = torch.cumsum(lens, 0)
    vals_out = None if binary else torch.cat([p[2] for p in per_group])[order].float().contiguous()
    space = ColumnSpace(torch.cat(space_keys) if space_keys else torch.zeros(0, dtype=torch.int64, device=dev),
                        space_groups, nnz_per_row, dropped)
    return cols[order].contiguous(), row_ptr.to(torch.int32), vals_out, space


@dataclass
class BlockPlan:
    blocks: List[Tuple[int, int]]               # column ranges, in column order
    group_of: List[int]                         # feature group of every block
    prior: List[int] = field(default_factory=list)      # block indices that open pass 0, one after another
    block_cols: int = 1                         # capacity the per-block exchange areas need


def plan_blocks(space: ColumnSpace, *, feature_block_ratio: float = 4.0, max_block_cols: int = 1 << 16,
                prior_groups: Sequence[int] = (), prior_iters: int = 5) -> BlockPlan:
    """Feature blocks as ``DarlinScheduler`` divides them (``app/linear_method/darlin.h:56-85``): group
    by group, ``ceil(nnz per row * feature_block_ratio)`` blocks of equal width (at least one; ratio 0:
    one block per group), never wider than ``max_block_cols`` columns. The blocks of the prior groups
    are listed ``prior_iters`` times to open the first pass."""
    blocks, group_of = [], []
    for (gid, c0, c1), nnzr in zip(space.groups, space.nnz_per_row):
        n = c1 - c0
        if n <= 0:
            continue
        want = max(1, math.ceil(nnzr * feature_block_ratio)) if feature_block_ratio > 0 else 1
        want = max(want, math.ceil(n / max_block_cols))
        want = min(want, n)
        for i in range(want):
            b0, b1 = c0 + n * i // want, c0 + n * (i + 1) // want
            if b1 > b0:
                blocks.append((b0, b1))
                group_of.append(gid)
    prior = []
    for gid in prior_groups:
        mine = [i for i, g in enumerate(group_of) if g == gid]
        prior += mine * max(1, prior_iters)
    cap = max([b1 - b0 for b0, b1 in blocks], default=1)
    return BlockPlan(blocks, group_of, prior, cap)
