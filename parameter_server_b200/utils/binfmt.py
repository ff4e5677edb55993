"""The raw binary matrix files of the reference's MATLAB helpers (``data/matlab/*.m``), in NumPy.

A matrix ``name`` is a handful of flat files: ``name.index`` (uint32 column of every nonzero,
row-major), ``name.offset`` (uint64 row offsets), ``name.value`` (float64 values, absent for binary
matrices), ``name.label`` (float64 labels) and a text ``name.info``. These functions read and write
them (``save_bin.m``, ``load_bin.m``, ``mat2bin.m``, ``bin2mat.m``), drop rare columns
(``filter_fea.m``) and write the parameter server's own text format (``saveas_pserver.m``).
"""
from __future__ import annotations

import re
from typing import Optional, Sequence, Tuple

import numpy as np
import scipy.sparse as sp


def save_bin(name: str, x, dtype="float64") -> int:
    a = np.ascontiguousarray(np.asarray(x).ravel(), dtype=dtype)
    a.tofile(name)
    return a.size


def load_bin(name: str, dtype="float64", offset: int = 0, length: Optional[int] = None) -> np.ndarray:
    dt = np.dtype(dtype)
    try:
        return np.fromfile(name, dtype=dt, count=-1 if length is None else int(length), offset=offset * dt.itemsize)
    except FileNotFoundError:
        return np.zeros(0, dtype=dt)


def mat2bin(name: str, y, X) -> None:
    """Label vector ``y`` and sparse matrix ``X`` (rows = examples) to ``name.{index,offset,value,label,info}``."""
    X = sp.csr_matrix(X)
    X.sort_indices()
    binary = bool(np.all((X.data == 0) | (X.data == 1)))
    save_bin(name + ".index", X.indices, "uint32")
    save_bin(name + ".offset", X.indptr, "uint64")
    if not binary:
        save_bin(name + ".value", X.data, "float64")
    save_bin(name + ".label", y, "float64")
    with open(name + ".info", "w") as f:
        f.write(f"type         : {'SPARSE_BINARY' if binary else 'SPARSE'}\n"
                "row_major    : true\nsparse       : true\n"
                f"bool_value   : {'true' if binary else 'false'}\n"
                f"row_begin    : 0\nrow_end      : {X.shape[0]}\ncol_begin    : 0\ncol_end      : {X.shape[1]}\n"
                f"entries      : {X.nnz}\nsizeof_index : 4\nsizeof_value : 8\n")


def _info(name: str) -> dict:
    out = {}
    with open(name + ".info") as f:
        for line in f:
            m = re.match(r"\s*(\w+)\s*:\s*(\S+)", line)
            if m:
                out.setdefault(m.group(1), []).append(m.group(2))
    return out


def bin2mat(name: str) -> Tuple[sp.csr_matrix, np.ndarray]:
    """``(X, y)`` back from the files written by :func:`mat2bin` (or by a converter that writes the same layout)."""
    info = _info(name)
    rows, cols = int(info["row_end"][0]), int(info["col_end"][0])
    indices = load_bin(name + ".index", "uint32").astype(np.int64)
    indptr = load_bin(name + ".offset", "uint64").astype(np.int64)
    binary = info.get("bool_value", ["false"])[0] == "true"
    data = np.ones(len(indices)) if binary else load_bin(name + ".value", "float64")
    X = sp.csr_matrix((data, indices, indptr), shape=(rows, cols))
    return X, load_bin(name + ".label", "float64")


def filter_fea(X, group_offset: Sequence[int], min_count: float = 4):
    """Drop the columns whose entries sum to ``min_count`` or less; returns the reduced matrix and the
    group offsets (first column of every feature group, plus the end) after the columns went away."""
    X = sp.csc_matrix(X)
    keep = np.asarray(X.sum(axis=0)).ravel() > min_count
    go = np.asarray(group_offset, dtype=np.int64)
    kept_before = np.concatenate([[0], np.cumsum(keep)])
    return X[:, keep].tocsr(), kept_before[go]


def saveas_pserver(file_name: str, y, X, group_id=None, binary: bool = False) -> None:
    """Text in the parameter server's ``label; group key[:value] ...;`` layout (``text: SPARSE`` or ``SPARSE_BINARY``)."""
    X = sp.csr_matrix(X)
    X.sort_indices()
    gid = np.zeros(X.shape[1], dtype=np.int64) if group_id is None else np.asarray(group_id, dtype=np.int64)
    assert np.all(np.diff(gid) >= 0), "group ids must be sorted by column"
    with open(file_name, "w") as f:
        for i in range(X.shape[0]):
            lo, hi = X.indptr[i], X.indptr[i + 1]
            parts = [f"{int(y[i])}"]
            prev = None
            for c, v in zip(X.indices[lo:hi], X.data[lo:hi]):
                if gid[c] != prev:
                    parts.append(f"; {gid[c]}")
                    prev = gid[c]
                parts.append(f" {c}" if binary else f" {c}:{v:g}")
            f.write("".join(parts) + ";\n")


BIN_SUFFIXES = (".index", ".offset", ".value", ".label", ".info")


def bin_base_names(files: Sequence[str]):
    """The matrices behind a list of file names: ``x.index, x.offset, x.info, ...`` and ``x`` all name ``x``."""
    out = []
    for f in files:
        for suf in BIN_SUFFIXES:
            if f.endswith(suf):
                f = f[:-len(suf)]
                break
        if f not in out:
            out.append(f)
    return out


class BinReader:
    """Minibatches straight from binary matrix files (``format: BIN`` in a data section), with the interface of
    the text / record stream reader: ``read_matrices(n)`` returns ``(labels, [csr dict])`` of the next ``n``
    rows or ``None`` at the end. Nothing is parsed: the files are mapped and a minibatch is a slice of them,
    which is what keeps a GPU fed (a text reader delivers some 10^4 rows/s per thread, this one 10^6 - 10^7).
    Indices are uint32 or uint64 (``sizeof_index`` in the ``.info`` file), values float32 or float64."""

    def __init__(self, files: Sequence[str]):
        self.names = bin_base_names(files)
        self.k = 0          # next matrix
        self.row = 0        # next row in the current one
        self.cur = None

    def _open(self, name: str):
        info = _info(name)
        isz = int(info.get("sizeof_index", ["4"])[0])
        vsz = int(info.get("sizeof_value", ["8"])[0])
        binary = info.get("bool_value", ["false"])[0] == "true"
        offset = np.memmap(name + ".offset", dtype=np.uint64, mode="r")
        nnz = int(offset[-1]) if len(offset) else 0
        m = dict(offset=offset, rows=len(offset) - 1, binary=binary,
                 index=np.memmap(name + ".index", dtype=np.uint32 if isz == 4 else np.uint64, mode="r") if nnz else np.zeros(0, np.uint64),
                 label=np.memmap(name + ".label", dtype=np.float64, mode="r"),
                 value=None if binary or not nnz else np.memmap(name + ".value", dtype=np.float32 if vsz == 4 else np.float64, mode="r"))
        return m

    def read_matrices(self, n: int):
        while True:
            if self.cur is None:
                if self.k >= len(self.names):
                    return None
                self.cur = self._open(self.names[self.k])
                self.k += 1
                self.row = 0
            m = self.cur
            if self.row >= m["rows"]:
                self.cur = None
                continue
            r0, r1 = self.row, min(m["rows"], self.row + int(n))
            self.row = r1
            o0, o1 = int(m["offset"][r0]), int(m["offset"][r1])
            k = o1 - o0
            # The arrays handed out are views of two sets of buffers used in turn (a minibatch stays valid
            # until the read after the next one): a fresh 100 MB array per minibatch would spend more time in
            # page faults than the copy takes.
            buf = self._buffers(r1 - r0, k)
            y = buf["y"][:r1 - r0]
            np.copyto(y, m["label"][r0:r1], casting="unsafe")
            off = buf["offset"][:r1 - r0 + 1]
            np.subtract(m["offset"][r0:r1 + 1], np.uint64(o0), out=off)
            idx = buf["index"][:k]
            np.copyto(idx, m["index"][o0:o1], casting="unsafe")
            if m["value"] is None:
                val = np.zeros(0, np.float32)
            else:
                val = buf["value"][:k]
                np.copyto(val, m["value"][o0:o1], casting="unsafe")
            return y, [dict(id=1, offset=off, index=idx, binary=m["binary"], value=val)]

    def _buffers(self, rows: int, nnz: int):
        self._turn = 1 - getattr(self, "_turn", 0)
        sets = self.__dict__.setdefault("_sets", [None, None])
        b = sets[self._turn]
        if b is None or len(b["y"]) < rows or len(b["index"]) < nnz:
            rows_cap = max(rows, len(b["y"]) if b else 0)
            nnz_cap = max(nnz + nnz // 8, len(b["index"]) if b else 0)
            b = sets[self._turn] = dict(y=np.empty(rows_cap, np.float32), offset=np.empty(rows_cap + 1, np.uint64),
                                        index=np.empty(nnz_cap, np.uint64), value=np.empty(nnz_cap, np.float32))
        return b


class BinWriter:
    """Appends minibatches (``(labels, [csr dict])`` as the readers return them) to one binary matrix with
    64-bit indices and float32 values: what ``datatool convert -to bin`` writes and :class:`BinReader` maps."""

    def __init__(self, name: str):
        self.name = name
        import os
        if os.path.dirname(name):
            os.makedirs(os.path.dirname(name), exist_ok=True)
        self.f = {k: open(name + "." + k, "wb") for k in ("index", "offset", "value", "label")}
        np.zeros(1, np.uint64).tofile(self.f["offset"])
        self.rows, self.nnz, self.binary, self.max_col = 0, 0, True, 0

    def add(self, batch) -> None:
        y, mats = batch
        m = mats[0]
        idx = np.ascontiguousarray(m["index"], dtype=np.uint64)
        off = np.asarray(m["offset"], dtype=np.uint64)
        np.asarray(y, dtype=np.float64).tofile(self.f["label"])
        idx.tofile(self.f["index"])
        (off[1:] + np.uint64(self.nnz)).tofile(self.f["offset"])
        if not m["binary"] and len(m["value"]):
            if self.binary and self.nnz:
                raise ValueError("binary and valued minibatches cannot be mixed in one matrix")
            self.binary = False
            np.asarray(m["value"], dtype=np.float32).tofile(self.f["value"])
        self.rows += len(y)
        self.nnz += len(idx)
        if len(idx):
            self.max_col = max(self.max_col, int(idx.max()))

    def close(self) -> None:
        for f in self.f.values():
            f.close()
        if self.binary:
            import os
            os.remove(self.name + ".value")
        with open(self.name + ".info", "w") as f:
            f.write(f"type         : {'SPARSE_BINARY' if self.binary else 'SPARSE'}\n"
                    "row_major    : true\nsparse       : true\n"
                    f"bool_value   : {'true' if self.binary else 'false'}\n"
                    f"row_begin    : 0\nrow_end      : {self.rows}\ncol_begin    : 0\ncol_end      : {self.max_col + 1}\n"
                    f"entries      : {self.nnz}\nsizeof_index : 8\nsizeof_value : 4\n")
