"""Binary shard checkpoints: every occupied table entry of one server shard
(key, weight and both optimiser state words) plus run metadata.

The reference only writes the final non-zero weights as text (``key<TAB>value``,
``parameter/kv_map.h:100-117``, ``app/linear_method/async_sgd.h:67-75``) and never
saves the FTRL ``z, n`` state; this is the binary extension that makes a run
resumable. One file per shard: ``<prefix>_S<rank>.psbckpt``.

Layout (little endian): magic ``PSBCKPT1`` | u32 header bytes | JSON header |
keys ``uint64[n]`` | w ``float32[n]`` | s0 ``float32[n]`` | s1 ``float32[n]``.
The header records n, rank, world, the shard's key range, the optimiser
configuration and free-form user metadata (e.g. the number of minibatches seen).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional, Tuple

import numpy as np

MAGIC = b"PSBCKPT1"


def shard_path(prefix: str, rank: int) -> str:
    return f"{prefix}_S{rank}.psbckpt"


def write_shard(path: str, keys: np.ndarray, w: np.ndarray, s0: np.ndarray, s1: np.ndarray,
                header: Dict[str, Any]) -> None:
    keys = np.ascontiguousarray(keys, dtype=np.uint64)
    arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (w, s0, s1)]
    n = int(keys.size)
    assert all(a.size == n for a in arrs)
    hdr = dict(header, n=n)
    hb = json.dumps(hdr, sort_keys=True).encode()
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(MAGIC)
        f.write(np.uint32(len(hb)).tobytes())
        f.write(hb)
        f.write(keys.tobytes())
        for a in arrs:
            f.write(a.tobytes())
    os.replace(tmp, path)     # a reader never sees a half-written file


def read_shard(path: str) -> Tuple[Dict[str, Any], np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError(f"{path}: not a shard checkpoint")
        (hl,) = np.frombuffer(f.read(4), dtype=np.uint32)
        hdr = json.loads(f.read(int(hl)).decode())
        n = int(hdr["n"])
        keys = np.frombuffer(f.read(8 * n), dtype=np.uint64).copy()
        w, s0, s1 = (np.frombuffer(f.read(4 * n), dtype=np.float32).copy() for _ in range(3))
        if keys.size != n or s1.size != n:
            raise ValueError(f"{path}: truncated")
    return hdr, keys, w, s0, s1


def save_plane(plane, prefix: str, meta: Optional[Dict[str, Any]] = None) -> str:
    """Write this rank's shard of a :class:`DataPlane`. Call it between steps (no
    kernels of the plane in flight)."""
    import torch
    torch.cuda.synchronize(plane.device)
    keys, s0, s1, w = plane.export_state()
    o = plane.opt
    hdr = {"rank": plane.rank, "world": plane.S,
           "key_begin": int(plane.bounds_host[plane.rank]), "key_end": int(plane.bounds_host[plane.rank + 1]),
           "optimizer": {k: getattr(o, k) for k in ("algo", "alpha", "beta", "l1", "l2") if hasattr(o, k)},
           "meta": meta or {}}
    path = shard_path(prefix, plane.rank)
    write_shard(path, keys, w.numpy(), s0.numpy(), s1.numpy(), hdr)
    return path


def load_plane(plane, prefix: str) -> Dict[str, Any]:
    """Load the entries of this rank's key range into a (fresh) plane. The checkpoint
    may have been written with a different number of shards: every shard file whose
    key range overlaps this rank's is read and filtered. Returns the user metadata
    of the first file read."""
    import torch
    lo, hi = int(plane.bounds_host[plane.rank]), int(plane.bounds_host[plane.rank + 1])
    meta = None
    r = 0
    found = False
    while os.path.exists(shard_path(prefix, r)):
        found = True
        hdr, keys, w, s0, s1 = read_shard(shard_path(prefix, r))
        r += 1
        if meta is None:
            meta = hdr.get("meta", {})
        if int(hdr["key_end"]) <= lo or int(hdr["key_begin"]) >= hi:
            continue
        m = (keys >= np.uint64(lo)) & (keys < np.uint64(hi)) if hi < (1 << 64) - 1 else (keys >= np.uint64(lo))
        if m.any():
            plane.load_state(keys[m], s0=torch.from_numpy(s0[m]), s1=torch.from_numpy(s1[m]), w=torch.from_numpy(w[m]))
    if not found:
        raise FileNotFoundError(shard_path(prefix, 0))
    plane.check_status("checkpoint load")
    return meta or {}
