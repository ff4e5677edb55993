"""CPU oracle: plain NumPy fp32 restatements of the math every kernel is checked
against. Same formulas as the reference: FTRL / AdaGrad entries
(``app/linear_method/async_sgd.h:132-176``), elastic-net proximal operator
(``app/linear_method/penalty.h:48-56``), learning rate
(``app/linear_method/learning_rate.h:15-22``), logistic loss and its gradient
(``app/linear_method/loss.h:81-93``).
"""
from __future__ import annotations

from typing import Dict

import numpy as np

f32 = np.float32

_M1 = np.uint64(0xff51afd7ed558ccd)
_M2 = np.uint64(0xc4ceb9fe1a85ec53)


def fmix64(k):
    k = np.asarray(k, dtype=np.uint64).copy()
    with np.errstate(over="ignore"):
        k ^= k >> np.uint64(33)
        k *= _M1
        k ^= k >> np.uint64(33)
        k *= _M2
        k ^= k >> np.uint64(33)
    return k


def hash_id_to_key(ids, seed: int, bits: int = 64):
    """Same map as the device ``hash_id_to_key`` (``bits`` significant key bits, in the top bits)."""
    ids = np.asarray(ids).astype(np.uint64)
    G = np.uint64(0x9E3779B97F4A7C15)
    with np.errstate(over="ignore"):
        if bits == 0 or bits >= 64:
            k = fmix64(ids + np.uint64(seed) * G + np.uint64(0x632BE59BD9B4E019))
            k[k == np.uint64(0xFFFFFFFFFFFFFFFF)] = np.uint64(0xFFFFFFFFFFFFFFFE)
            return k
        m = np.uint64((1 << bits) - 1)
        h = (ids + np.uint64(seed) * G) & m
        h = (h * _M1) & m
        h ^= h >> np.uint64(bits // 2)
        h = (h * _M2) & m
        h ^= h >> np.uint64(bits // 2 + 1)
        h = (h * G) & m
        h ^= h >> np.uint64(bits // 2)
        return h << np.uint64(64 - bits)


def lr_eval(opt, x):
    if opt.lr_type == "constant":
        return np.full_like(x, f32(opt.alpha), dtype=f32)
    return (f32(opt.alpha) / (x + f32(opt.beta))).astype(f32)


def prox(opt, z, eta):
    z, eta = z.astype(f32), eta.astype(f32)
    leta = f32(opt.l1) * eta
    den = f32(1) + f32(opt.l2) * eta
    out = np.where(z > 0, (z - leta) / den, (z + leta) / den).astype(f32)
    out[(z <= leta) & (z >= -leta)] = 0
    return out


def opt_step(opt, g, w, s0, s1):
    """Vectorised single optimiser step; returns new (w, s0, s1) as float32."""
    g, w, s0, s1 = (np.asarray(a, dtype=f32) for a in (g, w, s0, s1))
    if opt.algo == "ftrl":
        sn = np.sqrt(s1 * s1 + g * g).astype(f32)
        sigma = ((sn - s1) / f32(opt.alpha)).astype(f32)
        z = (s0 + (g - sigma * w)).astype(f32)
        eta = lr_eval(opt, sn)
        return prox(opt, -z * eta, eta), z, sn
    if opt.algo == "adagrad":
        s = (s0 + g * g).astype(f32)
        eta = lr_eval(opt, np.sqrt(s).astype(f32))
        return prox(opt, w - eta * g, eta), s, s1
    if opt.algo == "sgd":
        c = (s0 + f32(1)).astype(f32)
        eta = lr_eval(opt, np.sqrt(c).astype(f32))
        return prox(opt, w - eta * g, eta), c, s1
    return (w + g).astype(f32), s0, s1


def logit_loss_and_gcoef(y, margin):
    ym = (y * margin).astype(f32)
    en = np.exp(-np.abs(ym)).astype(f32)
    tau = np.where(ym > 0, en / (1 + en), 1 / (1 + en)).astype(f32)
    loss = (np.log1p(en) + np.maximum(-ym, 0)).astype(f32)
    return loss, (-y * tau).astype(f32)


class OracleTable:
    """Dictionary-backed server state keyed by uint64."""

    def __init__(self, opt):
        self.opt = opt
        self.idx: Dict[int, int] = {}
        self.w, self.s0, self.s1 = [], [], []

    def _slots(self, keys, insert=True):
        out = np.empty(len(keys), dtype=np.int64)
        for i, k in enumerate(keys.tolist()):
            j = self.idx.get(k, -1)
            if j < 0 and insert:
                j = len(self.w)
                self.idx[k] = j
                self.w.append(f32(0)); self.s0.append(f32(0)); self.s1.append(f32(0))
            out[i] = j
        return out

    def pull(self, keys):
        sl = self._slots(keys, insert=False)
        w = np.asarray(self.w + [f32(0)], dtype=f32)
        return w[sl]  # -1 -> appended zero

    def push(self, keys, grads):
        """keys unique; one optimiser step per key."""
        sl = self._slots(keys)
        w, s0, s1 = (np.asarray(a, dtype=f32) for a in (self.w, self.s0, self.s1))
        nw, n0, n1 = opt_step(self.opt, grads, w[sl], s0[sl], s1[sl])
        w[sl], s0[sl], s1[sl] = nw, n0, n1
        self.w, self.s0, self.s1 = list(w), list(s0), list(s1)

    def nonzero(self):
        items = sorted((k, self.w[j]) for k, j in self.idx.items() if self.w[j] != 0)
        return (np.array([k for k, _ in items], dtype=np.uint64),
                np.array([v for _, v in items], dtype=f32))


def localize(keys_flat):
    """(unique sorted keys, inverse column ids, counts)."""
    u, inv, cnt = np.unique(keys_flat, return_inverse=True, return_counts=True)
    return u, inv.astype(np.int64), cnt


def sparse_lr_step(table: OracleTable, keys_flat, row_ptr, y, vals=None):
    """One minibatch of sparse logistic regression against ``table``: pull,
    margins, loss, X^T g (minibatch sum, as ``async_sgd.h:286-292``), push."""
    u, col, _ = localize(keys_flat)
    w = table.pull(u)
    x = np.ones(len(keys_flat), dtype=f32) if vals is None else vals.astype(f32)
    contrib = (w[col] * x).astype(np.float64)
    margin = np.add.reduceat(contrib, row_ptr[:-1]).astype(f32) if len(keys_flat) else np.zeros(len(y), f32)
    loss, gc = logit_loss_and_gcoef(y.astype(f32), margin)
    rows = np.repeat(np.arange(len(y)), np.diff(row_ptr))
    grad = np.zeros(len(u), dtype=np.float64)
    np.add.at(grad, col, gc[rows].astype(np.float64) * x)
    table.push(u, grad.astype(f32))
    return float(loss.sum()), margin, u, grad.astype(f32)


def block_quantize(g, mode: str, group: int = 32):
    """Block-scaled quantise + dequantise of a value slice, as the push kernel
    does per group of ``group`` consecutive records of one (owner, source) inbox:
    int8: scale = amax/127, code = rint(v/scale); fp16: scale = amax, code = half(v/scale)."""
    g = np.asarray(g, dtype=f32)
    out = np.empty_like(g)
    for a in range(0, len(g), group):
        v = g[a:a + group]
        amax = f32(np.abs(v).max()) if len(v) else f32(0)
        if mode == "int8":
            scale = f32(amax / f32(127))
            code = np.rint((v / scale).astype(f32)) if amax > 0 else np.zeros_like(v)
            out[a:a + group] = (scale * np.clip(code, -127, 127).astype(f32)).astype(f32)
        elif mode == "fp16":
            scale = amax if amax > 0 else f32(1)
            out[a:a + group] = (scale * (v / scale).astype(np.float16).astype(f32)).astype(f32)
        else:
            out[a:a + group] = v
    return out


def auc(y, score):
    """Exact AUC by rank-sum (``util/evaluation.h:24-45``)."""
    y = np.asarray(y) > 0
    order = np.argsort(score, kind="stable")
    ranks = np.empty(len(score), dtype=np.float64)
    ranks[order] = np.arange(1, len(score) + 1)
    npos, nneg = y.sum(), (~y).sum()
    if npos == 0 or nneg == 0:
        return 0.5
    a = (ranks[y].sum() - npos * (npos + 1) / 2) / (npos * nneg)
    return float(a)


def darlin_oracle(parts, global_keys, lam, eta, delta_init, delta_max, blocks_per_pass, n_pass, kkt_ratio=10.0, tau=0, w0=None):
    """NumPy restatement of Darlin. ``parts``: list of (keys_flat uint64, row_ptr, y, vals or None) per
    worker; ``blocks_per_pass``: list (per pass) of lists of (c0, c1) column ranges in processing order.
    ``tau``: block delay: the gradient of the i-th block of a pass is taken before the weights of the
    blocks i - tau .. i - 1 reach the margins (0: every block sees all earlier ones).
    ``w0``: initial weight per global column (zero when None); the margins start at X w0.
    Returns (w per global column, history of objectives)."""
    ncol = len(global_keys)
    w = np.zeros(ncol, f32) if w0 is None else np.asarray(w0, f32).copy()
    delta = np.full(ncol, delta_init, f32); active = np.ones(ncol, bool)
    data = []
    for keys, row_ptr, y, vals in parts:
        col = np.searchsorted(global_keys, keys)
        rows = np.repeat(np.arange(len(y)), np.diff(row_ptr))
        x = np.ones(len(keys), f32) if vals is None else vals.astype(f32)
        m = np.zeros(len(y), f32)
        if w0 is not None:
            np.add.at(m, rows, w[col] * x)
        data.append(dict(col=col, rows=rows, x=x, y=y.astype(f32), m=m, binary=vals is None))
    n_ex = sum(len(d["y"]) for d in data)
    thr = 1e20
    hist = []

    def gradient(c0, c1):
        G = np.zeros(c1 - c0, np.float64); U = np.zeros(c1 - c0, np.float64)
        for d in data:
            sel = (d["col"] >= c0) & (d["col"] < c1) & active[d["col"]]
            c, r, x = d["col"][sel], d["rows"][sel], d["x"][sel]
            ym = d["y"][r] * d["m"][r]
            en = np.exp(-np.abs(ym)); t = np.where(ym > 0, en / (1 + en), 1 / (1 + en))
            dl = delta[c]
            if d["binary"]:
                g = -d["y"][r] * t; h = np.minimum(t * (1 - t) * np.exp(dl), 0.25)
            else:
                g = -d["y"][r] * t * x; h = np.minimum(t * (1 - t) * np.exp(np.abs(x) * dl), 0.25) * x * x
            np.add.at(G, c - c0, g); np.add.at(U, c - c0, h)
        return G, U

    def apply(c0, c1, G, U, thr):
        vio_max = 0.0
        new_w = w[c0:c1].copy()
        for j in range(c1 - c0):
            k = c0 + j
            if not active[k]:
                continue
            g, u = f32(G[j]), f32(U[j]) / f32(eta) + f32(1e-10)
            gp, gn = g + f32(lam), g - f32(lam)
            wk = w[k]; dd = -wk; vio = 0.0
            if wk == 0:
                if gp < 0: vio = -gp
                elif gn > 0: vio = gn
                elif gp > thr and gn < -thr:
                    active[k] = False; continue
            vio_max = max(vio_max, float(vio))
            if gp <= u * wk: dd = -gp / u
            elif gn >= u * wk: dd = -gn / u
            dd = min(delta[k], max(-delta[k], dd))
            delta[k] = min(delta_max, 2 * abs(dd) + 0.1)
            new_w[j] = wk + dd
        dw = new_w - w[c0:c1]
        for d in data:
            sel = (d["col"] >= c0) & (d["col"] < c1) & active[d["col"]]
            np.add.at(d["m"], d["rows"][sel], dw[d["col"][sel] - c0] * d["x"][sel])
        w[c0:c1] = new_w
        return vio_max

    for it in range(n_pass):
        vio_max = 0.0
        blocks = blocks_per_pass[it]
        waiting = {}
        for i in range(len(blocks) + tau):
            if i < len(blocks):
                waiting[i] = gradient(*blocks[i])
            if i >= tau:
                vio_max = max(vio_max, apply(*blocks[i - tau], *waiting.pop(i - tau), thr))
        loss = sum(float(np.sum(np.log1p(np.exp(-np.abs(d["y"] * d["m"]))) + np.maximum(-d["y"] * d["m"], 0))) for d in data)
        hist.append(loss + lam * float(np.abs(w).sum()))
        thr = vio_max / n_ex * kkt_ratio
    return w, hist
