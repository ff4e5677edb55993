"""Feature ids as a bit stream: ``bits`` bits per id, id ``i`` at bit offset ``i * bits`` of a little-endian
array of 32-bit words.

A loader that knows the largest id of its data set (the number of features) ships the ids of a minibatch
in ``ceil(log2(max_id + 1))`` bits each instead of 32 or 64: with 2^26 features that is 26 bits, 19 % fewer
bytes over PCIe for the one transfer that bounds the end-to-end rate. The device unpacks them to 32-bit
ids in one pass (``psb_unpack_ids``, ``csrc/cuda/datagen.cu``) at the start of the localisation.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


def bits_for(max_id: int) -> int:
    """Bits needed for ids in ``[0, max_id]`` (at least 1, at most 32)."""
    b = max(1, int(max_id).bit_length())
    assert b <= 32, "ids wider than 32 bits are sent as they are"
    return b


def pack_ids(ids, bits: int) -> np.ndarray:
    """Pack non-negative integer ids below ``2**bits`` into 32-bit words (returned as a uint32 array
    whose length is a multiple of 4, with one spare word, so that the device may read a word past the
    last id and copies stay 16-byte multiples)."""
    ids = np.ascontiguousarray(np.asarray(ids)).reshape(-1)
    n = ids.size
    assert 1 <= bits <= 32
    g = (n + 31) // 32
    v = np.zeros(g * 32, dtype=np.uint64)
    v[:n] = ids.astype(np.uint64)
    assert n == 0 or int(v.max()) < (1 << bits), "an id does not fit the given width"
    v = v.reshape(g, 32)
    words = np.zeros((g, bits), dtype=np.uint64)          # a group of 32 ids fills exactly `bits` words
    for j in range(32):
        off = j * bits
        w, sh = off >> 5, off & 31
        x = v[:, j] << np.uint64(sh)
        words[:, w] |= x & np.uint64(0xFFFFFFFF)
        if sh + bits > 32:
            words[:, w + 1] |= x >> np.uint64(32)
    flat = words.astype(np.uint32).reshape(-1)
    total = (flat.size + 1 + 3) // 4 * 4
    out = np.zeros(total, dtype=np.uint32)
    out[:flat.size] = flat
    return out


def unpack_ids(words: np.ndarray, bits: int, n: int) -> np.ndarray:
    """NumPy inverse of :func:`pack_ids` (the restatement the device kernel is tested against)."""
    words = np.asarray(words, dtype=np.uint32).astype(np.uint64)
    i = np.arange(n, dtype=np.uint64)
    off = i * np.uint64(bits)
    w, sh = (off >> np.uint64(5)).astype(np.int64), off & np.uint64(31)
    two = words[w] | (words[w + 1] << np.uint64(32))
    return ((two >> sh) & np.uint64((1 << bits) - 1)).astype(np.uint32)


@dataclass
class PackedIds:
    """Packed ids of one minibatch: ``words`` (int32 tensor, host pinned or device), ``bits`` per id, ``n`` ids."""
    words: torch.Tensor
    bits: int
    n: int

    @classmethod
    def from_ids(cls, ids, bits: int, pin: bool = True) -> "PackedIds":
        arr = ids.cpu().numpy() if isinstance(ids, torch.Tensor) else np.asarray(ids)
        t = torch.from_numpy(pack_ids(arr, bits).view(np.int32))
        return cls(t.pin_memory() if pin and torch.cuda.is_available() else t, bits, int(arr.size))

    def numel(self) -> int:
        return self.n

    @property
    def is_cuda(self) -> bool:
        return self.words.is_cuda

    def nbytes(self) -> int:
        return self.words.numel() * 4
