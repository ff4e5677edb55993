"""Synthetic sparse-LR minibatches (device generator + host pools)."""
from __future__ import annotations

import torch

from ..ops import _lib
from ..ops._lib import check, ptr, stream_ptr


def gen_batch(n_rows: int, z: int, n_feat: int, zipf_s: float, seed: int, batch: int, *,
              device="cuda", ids64: bool = False, real_values: bool = False):
    """One minibatch on the device: ``(ids, y, vals)``; ids are raw feature ids
    (int32, or int64 when ``ids64``), ``vals`` is None for binary features."""
    dev = torch.device(device)
    ids = torch.empty(n_rows * z, dtype=torch.int64 if ids64 else torch.int32, device=dev)
    y = torch.empty(n_rows, dtype=torch.float32, device=dev)
    vals = torch.empty(n_rows * z, dtype=torch.float32, device=dev) if real_values else None
    check(_lib.lib().psb_gen_batch(0 if ids64 else ptr(ids), ptr(ids) if ids64 else 0, ptr(vals), ptr(y),
                                   n_rows, z, n_feat, zipf_s, seed, batch, int(real_values),
                                   stream_ptr()), "gen_batch")
    return ids, y, vals


def flush_l2(buf: torch.Tensor, value: int = 0):
    """Overwrite ``buf`` (int32, larger than L2) to evict L2 between timed iterations."""
    check(_lib.lib().psb_flush_l2(ptr(buf), buf.numel(), value, stream_ptr()), "flush_l2")
