"""Device filters and sorted-key utilities (kernels in ``csrc/cuda/filters.cu``)."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, ptr, stream_ptr


def fixing_float_encode(x: torch.Tensor, num_bytes: int = 3, lo: float | None = None, hi: float | None = None,
                        seed: int = 0):
    """Reference fixed-point codec: returns ``(codes uint8[n*num_bytes], lo, hi)``.
    ``lo``/``hi`` default to the data's min and max+1e-6 (computed on the device)."""
    x = x.contiguous().float()
    if lo is None or hi is None:
        mm = torch.tensor([float("inf"), float("-inf")], device=x.device)
        check(_lib.lib().psb_minmax(ptr(x), x.numel(), ptr(mm), stream_ptr()), "minmax")
        mn, mx = mm.tolist()
        lo = mn if lo is None else lo
        hi = mx + 1e-6 if hi is None else hi
    code = torch.empty(x.numel() * num_bytes, dtype=torch.uint8, device=x.device)
    check(_lib.lib().psb_fixfloat_encode(ptr(x), ptr(code), x.numel(), num_bytes, lo, hi, seed, stream_ptr()),
          "fixfloat_encode")
    return code, lo, hi


def fixing_float_decode(code: torch.Tensor, num_bytes: int, lo: float, hi: float) -> torch.Tensor:
    n = code.numel() // num_bytes
    out = torch.empty(n, dtype=torch.float32, device=code.device)
    check(_lib.lib().psb_fixfloat_decode(ptr(code), ptr(out), n, num_bytes, lo, hi, stream_ptr()), "fixfloat_decode")
    return out


def add_noise(x: torch.Tensor, mean: float, std: float, seed: int = 0):
    check(_lib.lib().psb_add_noise(ptr(x), x.numel(), mean, std, seed, stream_ptr()), "add_noise")
    return x


class CountMin:
    """Count-min sketch with saturating uint8 cells on the device; same hash and
    probe sequence as the host ``CountMin`` (sketch contents are identical)."""

    def __init__(self, n: int, k: int, device="cuda"):
        self.n, self.k = max(n, 64), min(30, max(1, k))
        self.cells = torch.zeros((self.n + 3) // 4, dtype=torch.int32, device=device)

    def insert(self, keys: torch.Tensor, counts: torch.Tensor | None = None, n_ptr: torch.Tensor | None = None):
        check(_lib.lib().psb_countmin_insert(ptr(self.cells), self.n, self.k, ptr(keys), ptr(counts), ptr(n_ptr),
                                             keys.numel(), stream_ptr()), "countmin_insert")

    def query(self, keys: torch.Tensor, n_ptr: torch.Tensor | None = None) -> torch.Tensor:
        out = torch.zeros(keys.numel(), dtype=torch.uint8, device=keys.device)
        check(_lib.lib().psb_countmin_query(ptr(self.cells), self.n, self.k, ptr(keys), ptr(out), ptr(n_ptr),
                                            keys.numel(), stream_ptr()), "countmin_query")
        return out

    def bytes(self) -> torch.Tensor:
        return self.cells.view(torch.uint8)[:self.n]


def ordered_match(src_key: torch.Tensor, src_val: torch.Tensor, dst_key: torch.Tensor, dst_val: torch.Tensor,
                  k: int = 1, op: int = 0) -> int:
    """``dst_val[j] op= src_val[i]`` for every ``src_key[i] == dst_key[j]`` (both
    sorted unique, int64-viewed uint64). ``op``: 0 assign, 1 plus, 2 minus, 3 times,
    4 divide. Returns the number of matched keys."""
    m = torch.zeros(1, dtype=torch.int64, device=src_key.device)
    check(_lib.lib().psb_ordered_match(ptr(src_key), ptr(src_val), src_key.numel(), ptr(dst_key), ptr(dst_val),
                                       dst_key.numel(), k, op, ptr(m), stream_ptr()), "ordered_match")
    return int(m.item())
