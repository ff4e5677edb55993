"""Small synthetic data sets written in the text formats the parsers read."""
from __future__ import annotations

import os
from typing import List, Tuple

import numpy as np


def write_sparse_binary(dirname: str, n_files: int, rows_per_file: int, nnz: int, n_feat: int, *, seed: int = 0,
                        zipf_s: float = 1.1, w_density: float = 0.05, prefix: str = "part") -> Tuple[List[str], np.ndarray]:
    """Files ``<dirname>/<prefix>-NN`` in the native SPARSE_BINARY text format
    (``label; group key key ...;``). Ids follow a Zipf-like law and are spread
    over the uint64 key space by a multiplicative hash so that key-range shards
    are balanced. Labels are ``sign(x.w* + logistic noise)`` with a sparse ``w*``.
    Returns the file list and the dense ground truth (indexed by id)."""
    rng = np.random.default_rng(seed)
    w_star = np.where(rng.random(n_feat) < w_density, rng.normal(0, 1.5, n_feat), 0.0)
    os.makedirs(dirname, exist_ok=True)
    files = []
    for f in range(n_files):
        ids = np.minimum((rng.pareto(zipf_s, (rows_per_file, nnz)) * 3).astype(np.int64), n_feat - 1)
        ids = np.sort(ids, axis=1)
        margin = w_star[ids].sum(axis=1)
        u = rng.random(rows_per_file)
        y = np.where(margin + np.log(u / (1 - u)) >= 0, 1, -1)
        keys = key_of_id(ids)
        name = os.path.join(dirname, f"{prefix}-{f:02d}")
        with open(name, "w") as out:
            for r in range(rows_per_file):
                ks = np.unique(keys[r])
                out.write(f"{y[r]}; 1 " + " ".join(map(str, ks.tolist())) + ";\n")
        files.append(name)
    return files, w_star


def key_of_id(ids):
    """Feature id -> uint64 key (odd multiplicative hash: a bijection)."""
    with np.errstate(over="ignore"):
        return (np.asarray(ids).astype(np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)


def write_libsvm(dirname: str, n_files: int, rows_per_file: int, nnz: int, n_feat: int, *, seed: int = 0,
                 w_density: float = 0.05, prefix: str = "part") -> Tuple[List[str], np.ndarray]:
    """Files in LIBSVM format (``label index:value ...``, indices ascending, real values): the format of
    the reference's rcv1 example. Labels are ``sign(x.w* + logistic noise)`` with a sparse ``w*``."""
    rng = np.random.default_rng(seed)
    w_star = np.where(rng.random(n_feat) < w_density, rng.normal(0, 1.5, n_feat), 0.0)
    os.makedirs(dirname, exist_ok=True)
    files = []
    for f in range(n_files):
        name = os.path.join(dirname, f"{prefix}-{f:02d}")
        with open(name, "w") as out:
            for _ in range(rows_per_file):
                ids = np.unique(np.minimum((rng.pareto(1.1, nnz) * 3).astype(np.int64), n_feat - 1))
                x = np.round(rng.random(len(ids)) + 0.1, 4)
                u = rng.random()
                y = 1 if float(w_star[ids] @ x) + np.log(u / (1 - u)) >= 0 else -1
                out.write(f"{y} " + " ".join(f"{i + 1}:{v}" for i, v in zip(ids.tolist(), x.tolist())) + "\n")
        files.append(name)
    return files, w_star


def write_criteo(dirname: str, n_files: int, rows_per_file: int, *, seed: int = 0, prefix: str = "part") -> List[str]:
    """Files in the Criteo click-log format (``label<TAB>13 integer features<TAB>26 categorical features``
    as 8-digit hex strings, some fields empty): the format of the reference's criteo example. The
    label depends on a few of the categorical fields."""
    rng = np.random.default_rng(seed)
    os.makedirs(dirname, exist_ok=True)
    weight = np.random.default_rng(12345).normal(0, 1.0, (26, 40))     # the same ground truth for every seed
    files = []
    for f in range(n_files):
        name = os.path.join(dirname, f"{prefix}-{f:02d}")
        with open(name, "w") as out:
            for _ in range(rows_per_file):
                ints = [str(int(v)) if rng.random() > 0.1 else "" for v in rng.poisson(3, 13)]
                cats = np.minimum((rng.pareto(1.2, 26) * 2).astype(np.int64), 39)
                score = float(weight[np.arange(26), cats][:6].sum())
                u = rng.random()
                y = 1 if score + np.log(u / (1 - u)) >= 0 else 0
                cat_s = [f"{(int(c) * 2654435761 + k * 97) & 0xffffffff:08x}" if rng.random() > 0.05 else ""
                         for k, c in enumerate(cats)]
                out.write("\t".join([str(y)] + ints + cat_s) + "\n")
        files.append(name)
    return files
