"""Half-open key ranges and the even partition of the key space over servers.

Mirrors ``Range<T>`` of the reference (``util/range.h:10-131``); the even
division uses 80-bit extended arithmetic exactly like ``Range::EvenDivide``
(``util/range.h:99-107``) so that server boundaries agree bit for bit.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

K_MAX_KEY = (1 << 64) - 1  # exclusive end of the full key space; never a valid key


@dataclass(frozen=True)
class Range:
    begin: int = 0
    end: int = K_MAX_KEY

    @staticmethod
    def all() -> "Range":
        return Range(0, K_MAX_KEY)

    def valid(self) -> bool:
        return self.end >= self.begin

    def empty(self) -> bool:
        return self.begin >= self.end

    def size(self) -> int:
        return self.end - self.begin

    def contains(self, other) -> bool:
        if isinstance(other, Range):
            return self.begin <= other.begin and other.end <= self.end
        return self.begin <= other < self.end

    def set_intersection(self, o: "Range") -> "Range":
        return Range(max(self.begin, o.begin), min(self.end, o.end))

    def set_union(self, o: "Range") -> "Range":
        return Range(min(self.begin, o.begin), max(self.end, o.end))

    def project(self, v: int) -> int:
        return max(self.begin, min(self.end, v))

    def even_divide(self, n: int, i: int) -> "Range":
        assert self.valid() and n > 0 and 0 <= i < n
        ld = np.longdouble
        itv = ld(self.end - self.begin) / ld(n)
        lo = int(ld(self.begin) + itv * ld(i))
        hi = self.end if i + 1 == n else int(ld(self.begin) + itv * ld(i + 1))
        return Range(lo, hi)

    def __add__(self, v: int) -> "Range":
        return Range(self.begin + v, self.end + v)

    def __str__(self) -> str:
        return f"[{self.begin},{self.end})"


def shard_bounds(key_range: Range, n: int):
    """``n+1`` boundaries; shard ``s`` owns ``[b[s], b[s+1])``."""
    b = [key_range.even_divide(n, i).begin for i in range(n)]
    b.append(key_range.end)
    return b
