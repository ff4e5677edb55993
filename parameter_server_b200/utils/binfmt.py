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
