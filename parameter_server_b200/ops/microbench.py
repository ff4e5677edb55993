"""Per-kernel micro-benchmarks with CUDA-event timing and roofline fractions.

    python -m parameter_server_b200.ops.microbench sort  --n 13107200
    python -m parameter_server_b200.ops.microbench step  --rows 65536 --z 200

Each timed launch is preceded by an L2 flush (a write over a 256 MB buffer) and
timed with CUDA events on the launching stream after warm-up. Fractions are
"of measured": the denominators come from ``MEASURED_PEAKS.json`` at the
repository root when present (copy bandwidth), else 6650 GB/s ("of fallback").
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
from pathlib import Path

import torch


def _peak_gbs():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())["hbm_gbs"], "of measured"
    return 6650.0, "of fallback"


def _time(fn, iters, flush):
    from ..utils.synthetic import flush_l2
    ts = []
    for i in range(iters + 3):
        flush_l2(flush, i)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        if i >= 3:
            ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_sort(args):
    from . import _lib
    from .localize import LocalBatch
    from ..utils.synthetic import gen_batch
    n = args.n
    dev = torch.device("cuda")
    flush = torch.empty(64 << 20, dtype=torch.int32, device=dev)
    ids, _, _ = gen_batch(n // 200, 200, 1 << 26, 1.05, 0, 0, device=dev)
    n = ids.numel()
    b = LocalBatch(n // 200, n, 1, dev)
    bounds = torch.tensor([0, -1], dtype=torch.int64, device=dev)
    peak, tag = _peak_gbs()

    def run():
        b.localize(ids, None, bounds, fixed_z=200, hash_seed=0, hash_bits=args.bits % 64)
    med, best = _time(run, args.iters, flush)
    _lib.check_status(b.status, "sort")
    npass = (args.bits + 7) // 8     # digit passes that are not skipped
    bytes_sort = n * (4 + 8 + 8) + npass * n * 24       # ids read + keys write + hist read; passes r+w
    print(json.dumps({"kernel": "sort+localize", "n": n, "passes": npass, "ms_median": med, "ms_best": best,
                      "sort_algorithmic_GB": bytes_sort / 1e9,
                      "frac_of_copy_bw_if_all_sort": bytes_sort / 1e9 / (med * 1e-3) / peak, "peak": tag}))


def bench_localize(args):
    """The localisation of one minibatch alone (unique keys + CSC/CSR remap + owner offsets) on
    ``--rows`` x ``--z`` ids hashed to ``--key-bits`` significant bits: milliseconds per call by CUDA
    events over distinct minibatches (inputs larger than L2), for ``--method`` bucket, sort or auto, and
    with ``--graph`` replayed from a CUDA graph. Small ``--iters`` / ``--warmup`` make it a profiler target."""
    from ..ops.localize import LocalBatch
    from ..utils.synthetic import gen_batch
    dev = torch.device("cuda")
    rows, z = args.rows, args.z
    nnz = rows * z
    pool = [gen_batch(rows, z, 1 << args.log2_keys, 1.05, 0, i, device=dev)[:2] for i in range(4)]
    b = LocalBatch(rows, nnz, 1, dev)
    bounds = torch.tensor([0, -1], dtype=torch.int64, device=dev)
    kw = dict(fixed_z=z, hash_seed=0, hash_bits=args.key_bits % 64, method=args.method)
    st = torch.cuda.Stream(device=dev)          # a graph cannot be captured on the default stream

    def run(i):
        ids, y = pool[i % len(pool)]
        if args.graph:
            b.localize_replayed(ids, y, bounds, stream=st, **kw)
        else:
            b.localize(ids, y, bounds, stream=st, **kw)
    with torch.cuda.stream(st):
        for i in range(max(args.warmup, 2 * len(pool) if args.graph else 0)):   # every minibatch through its capture
            run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        e0.record(st)
        for i in range(args.iters):
            run(i)
        e1.record(st)
    torch.cuda.synchronize()
    _lib_check = int(b.status.item())
    print(json.dumps({"kernel": "localize", "rows": rows, "z": z, "nnz": nnz, "key_bits": args.key_bits, "method": args.method,
                      "graph": bool(args.graph), "unique": int(b.n_unique.item()), "fell_back_to_sort": int(b.gate.item()),
                      "status": _lib_check, "ms": round(e0.elapsed_time(e1) / max(1, args.iters), 4)}))


def bench_step(args):
    from . import _lib
    from ..models.sparse_lr import SparseLRConfig, make_single_gpu
    from ..parallel.dataplane import OptimizerConfig
    from ..utils.synthetic import gen_batch
    dev = torch.device("cuda")
    rows, z = args.rows, args.z
    nnz = rows * z
    cap = 1
    while cap < 2 * (1 << args.log2_keys):
        cap *= 2
    w = make_single_gpu(cap, nnz, OptimizerConfig(), SparseLRConfig(max_rows=rows, max_nnz=nnz, pipeline=1, hash_bits=40),
                        dev, ordered_slots=not args.hashed_slots, pull_cap=nnz)
    flush = torch.empty(64 << 20, dtype=torch.int32, device=dev)
    pool = [gen_batch(rows, z, 1 << args.log2_keys, 1.05, 0, i, device=dev)[:2] for i in range(3)]
    peak, tag = _peak_gbs()
    plane = w.plane
    state = {"t": 0}
    # warm the table so that pulls hit existing entries
    for ids, y in pool:
        w.step(ids, y, fixed_z=z)
    torch.cuda.synchronize()
    b = w.prepare(*pool[0], fixed_z=z, slot=0)
    U = int(b.n_unique.item())
    res = {"rows": rows, "z": z, "nnz": nnz, "unique": U, "peak": tag}

    def t_prep():
        w.prepare(*pool[0], fixed_z=z, slot=0)

    def t_pull():
        plane.pull_exchange(b, w.step_no, need_applied=0)

    def t_push():
        plane.push(b, w.step_no, send_keys=False)

    def t_apply():
        plane.apply(w.step_no)
        w.step_no += 1
    for name, fn, alg_bytes in (
            ("localize(sort+unique+remap)", t_prep, nnz * 20 + 8 * nnz * 24 + nnz * 8 * 2 + nnz * 12),
            ("pull_exchange", t_pull, U * (8 + 8 + 8 + 32 + 4 + 4 + 4) + nnz * 8 + rows * 12),
            ("push", t_push, nnz * 8 + U * (4 + 4 + 4)),
            ("apply", t_apply, U * (4 + 4 + 64))):
        if name == "apply":
            # every apply needs a fresh push of the same round
            from ..utils.synthetic import flush_l2
            ts = []
            for i in range(args.iters + 2):
                plane.pull_exchange(b, w.step_no, need_applied=0)
                plane.push(b, w.step_no, send_keys=False)
                flush_l2(flush, i)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record(); torch.cuda.synchronize()
                if i >= 2:
                    ts.append(e0.elapsed_time(e1))
            ts.sort(); med = ts[len(ts) // 2]
        elif name == "push":
            from ..utils.synthetic import flush_l2
            ts = []
            for i in range(args.iters + 2):
                plane.pull_exchange(b, w.step_no, need_applied=0)   # zeroes grad, fills the slot cache
                flush_l2(flush, i)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record(); torch.cuda.synchronize()
                plane.apply(w.step_no); w.step_no += 1
                if i >= 2:
                    ts.append(e0.elapsed_time(e1))
            ts.sort(); med = ts[len(ts) // 2]
        else:
            med, _ = _time(fn, args.iters, flush)
        res[name] = {"ms": med, "algorithmic_MB": alg_bytes / 1e6,
                     "frac_of_copy_bw": alg_bytes / 1e9 / (med * 1e-3) / peak}
    plane.check_status("microbench")
    print(json.dumps(res))


def bench_wide(args):
    """Wide-value pull fused with the tcgen05 GEMM against the context matrix."""
    from . import _lib
    from .localize import LocalBatch
    from ..parallel.fabric import Fabric
    from ..parallel.wide import WideConfig, WidePlane, wide_layout
    from ..utils.synthetic import gen_batch
    import numpy as np
    dev = torch.device("cuda")
    rows, z, N = args.rows, args.z, args.n_ctx
    cap = 1
    while cap < 2 * (1 << args.log2_keys):
        cap *= 2
    cfg = WideConfig(table_capacity=cap, inbox_cap=rows * z, ring=2)
    fab = Fabric.single(wide_layout(cfg, 1).total())
    plane = WidePlane(fab, cfg)
    ids, y, _ = gen_batch(rows, z, 1 << args.log2_keys, 1.2, 0, 0, device=dev)
    b = LocalBatch(rows, rows * z, 1, dev)
    b.localize(ids, y, plane.bounds, fixed_z=z, hash_seed=0, hash_bits=40)
    torch.cuda.synchronize()
    U = int(b.n_unique.item())
    # put every key of the batch into the table with random rows
    plane.load(b.ukeys[:U].cpu().numpy().view(np.uint64), torch.randn(U, 64) * 0.1)
    ctx = (torch.randn(N, 64) * 0.3).to(torch.bfloat16).to(dev)
    P = torch.zeros(rows * z, N, device=dev)
    flush = torch.empty(64 << 20, dtype=torch.int32, device=dev)
    peak, tag = _peak_gbs()
    med, best = _time(lambda: plane.pull_gemm(b, ctx, P), args.iters, flush)
    plane.check_status("wide")
    # bytes: key list + key-table probes (8 B) + value rows (128 B) + result (N*4 B)
    alg = U * (8 + 8 + 128 + N * 4)
    print(json.dumps({"kernel": "wide_pull_gemm", "unique_keys": U, "N": N, "ms_median": med, "ms_best": best,
                      "algorithmic_MB": alg / 1e6, "frac_of_copy_bw": alg / 1e9 / (med * 1e-3) / peak,
                      "tflops": 2.0 * U * 64 * N / (med * 1e-3) / 1e12, "peak": tag}))


def bench_wide_step(args):
    """Full training step of the wide-value model on 1..N ranks: localise, pull fused with
    the tcgen05 product against the batch's context matrix, row sums + loss, push of
    64-wide bf16 gradients to the owners, AdaGrad apply. Per worker `rows` x `z` keys
    (Zipf s = 1.2) over 2^log2_keys ids; examples/s of the whole job, max over ranks."""
    import numpy as np
    import torch.distributed as dist
    from .localize import LocalBatch
    from ..parallel.fabric import Fabric
    from ..parallel.wide import WideConfig, WidePlane, wide_layout
    from ..utils.synthetic import gen_batch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rows, z, N = args.rows, args.z, args.n_ctx
    n_feat = 1 << args.log2_keys
    cap = 1
    while cap < 2 * n_feat // world:
        cap *= 2
    cfg = WideConfig(table_capacity=cap, inbox_cap=rows * z, ring=args.tau + 2, pull_cap=0 if args.one_sided else rows * z)
    hb = wide_layout(cfg, world).total()
    fab = Fabric.from_process_group(hb) if world > 1 else Fabric.single(hb)
    plane = WidePlane(fab, cfg)
    pool = [gen_batch(rows, z, n_feat, 1.2, 0, rank * 1009 + i, device=dev)[:2] for i in range(args.pool)]
    bufs = [LocalBatch(rows, rows * z, world, dev) for _ in range(2)]
    # every key of every rank's pool goes into its owner's table before timing
    mine = []
    for ids, y in pool:
        b = bufs[0].localize(ids, y, plane.bounds, fixed_z=z, hash_seed=0, hash_bits=40)
        torch.cuda.synchronize()
        mine.append(b.ukeys[:int(b.n_unique.item())].cpu().numpy().view(np.uint64).copy())
    allk = [np.unique(np.concatenate(mine))]
    if world > 1:
        got = [None] * world
        dist.all_gather_object(got, allk[0])
        allk = got
    lo, hi = plane.bounds_host[rank], plane.bounds_host[rank + 1]
    own = np.unique(np.concatenate([k[(k >= np.uint64(lo)) & ((k < np.uint64(hi)) if hi < (1 << 64) - 1 else True)] for k in allk]))
    g = torch.Generator().manual_seed(rank)
    for c0 in range(0, len(own), 1 << 20):
        kk = own[c0:c0 + (1 << 20)]
        plane.load(kk, torch.randn(len(kk), 64, generator=g) * 0.1)
    ctx = (torch.randn(N, 64, generator=torch.Generator().manual_seed(7)) * 0.3).to(torch.bfloat16).to(dev)
    P = torch.zeros(rows * z, N, device=dev)
    step_no = [0]

    def pull_and_rows(b, mark=lambda: None):
        """Default: the pull kernel stores the product matrix P[U x N] and a second kernel gathers per row.
        --fused: the pull kernel adds the products into the rows' margins itself and nothing of P reaches
        memory (less traffic; at this size the extra work per tile costs more than the traffic it saves)."""
        fused = args.fused
        if cfg.pull_cap:
            plane.pull_xgemm(b, ctx, None if fused else P, step_no[0], fuse_margins=fused)
        else:
            plane.pull_gemm(b, ctx, None if fused else P, fuse_margins=fused)
        mark()
        if fused:
            plane.rowloss(b)
        else:
            plane.rowsum(b, P, N)

    def step(i):
        ids, y = pool[i % len(pool)]
        b = bufs[i % 2].localize(ids, y, plane.bounds, fixed_z=z, hash_seed=0, hash_bits=40)
        pull_and_rows(b)
        plane.push(b, ctx, step_no[0])
        plane.apply(step_no[0])
        step_no[0] += 1

    for i in range(4):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.iters):
        step(i)
    e1.record(); torch.cuda.synchronize()
    plane.check_status("wide step")
    # stage times (CUDA events, stages back to back on one stream), a few steps
    names = ["localize", "pull_gemm", "rowsum", "push", "apply"]
    acc = [0.0] * 5
    for i in range(6):
        ids, y = pool[i % len(pool)]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        ev[0].record()
        b = bufs[i % 2].localize(ids, y, plane.bounds, fixed_z=z, hash_seed=0, hash_bits=40)
        ev[1].record()
        pull_and_rows(b, ev[2].record)
        ev[3].record(); plane.push(b, ctx, step_no[0])
        ev[4].record(); plane.apply(step_no[0])
        ev[5].record(); step_no[0] += 1
        torch.cuda.synchronize()
        for k in range(5):
            acc[k] += ev[k].elapsed_time(ev[k + 1]) / 6
    if world > 1:
        ta = torch.tensor(acc, dtype=torch.float64, device=dev)
        dist.all_reduce(ta, op=dist.ReduceOp.MAX)
        acc = ta.tolist()
    stages = {n: round(v, 4) for n, v in zip(names, acc)}
    ms = e0.elapsed_time(e1) / args.iters
    u = float(np.mean([len(k) for k in mine]))
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    st = plane.stats.cpu().tolist()
    if rank == 0:
        print(json.dumps({"kernel": "wide model training step", "gpus": world, "rows_per_gpu": rows, "keys_per_row": z,
                          "table_keys": n_feat, "contexts": N, "unique_keys_per_step_per_gpu": u, "ms_per_step": ms,
                          "examples_per_s": world * rows / (ms * 1e-3),
                          "value_bytes_pulled_and_pushed_per_s": world * u * 256 / (ms * 1e-3),
                          "loss_per_example": st[0] / max(1.0, st[2]), "stage_ms_max_over_ranks": stages}))
    if world > 1:
        dist.barrier(); fab.close(); dist.destroy_process_group()


def bench_kv(args):
    """Push + pull of K sorted unique keys per rank through the device KV containers, for value widths
    ``--widths`` and filters ``--modes`` (``none``; ``key_caching``: the key list repeats, so after the
    first round no keys travel; ``int8``: block-scaled 8-bit values on the wire): milliseconds for the
    pair push-then-pull (max over ranks) and keys/s over all ranks. Under torch.distributed.run every
    rank is a worker and owns one key-range shard. ``nccl_ms`` is the same pair done the conventional
    way on the same table (all-to-all-v of keys and values through NCCL, then look-up and merge by the
    owner with the library's kernels, ``parallel/nccl_baseline.py`` ``NcclKV``); its split sizes are
    computed once outside the timed region. ``max_err`` compares what the last pull returned with the
    sum of everything pushed. The reference's probe: ``test/kv_map_perf_ps.cc:27-60``."""
    import numpy as np
    import torch.distributed as dist
    from ..parallel.dataplane import OptimizerConfig
    from ..parallel.nccl_baseline import NcclKV
    from ..parameter.kv import DeviceKVVector
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    modes = [args.quant] if args.quant != "none" and args.modes == ["none"] else args.modes
    out = []

    def timed(fn, reps, finish=lambda: None):
        for _ in range(3):
            fn()
        finish()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        finish()                                   # the containers work on a stream of their own
        e1.record(); torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for K in args.sizes:
        rng = np.random.default_rng(K + rank)
        keys = np.unique(rng.integers(0, 1 << 63, int(K * 1.2), dtype=np.uint64) * np.uint64(2))[:K]
        kt = torch.from_numpy(keys.view(np.int64)).to(dev)
        for width in args.widths:
            if K * width > args.max_values:
                continue                                      # the inbox ring would not fit
            vals = torch.randn(len(keys), width, device=dev)
            for mode in modes:
                cap = 1 << max(12, int(np.ceil(np.log2(4 * K))))
                kv = DeviceKVVector.create(None, table_capacity=cap, max_keys=K, opt=OptimizerConfig(algo="sum"),
                                           quant=mode if mode in ("int8", "fp16") else "none", k=width,
                                           key_cache=mode == "key_caching", exchange=not args.one_sided)
                fab = kv.plane.fabric
                pushes = [0]
                last = [None]

                def pair():
                    pushes[0] += 1
                    if last[0] is not None:
                        kv.discard(last[0])
                    last[0] = kv.pull(kt, wait=[kv.push(kt, vals)])

                ms = timed(pair, args.iters, lambda: kv.stream.synchronize())
                kv.wait(last[0])
                got = kv.result(last[0]).view(len(keys), width)
                err = float((got - pushes[0] * vals).abs().max().item() / pushes[0])
                row = {"K_per_rank": len(keys), "width": width, "mode": mode, "ms_push_pull": round(ms, 4),
                       "keys_per_s": 2 * len(keys) * world / (ms * 1e-3),
                       "value_GB_per_s": 2 * len(keys) * width * 4 * world / (ms * 1e-3) / 1e9,
                       "max_err": err, "nccl_ms": None}
                if args.nccl and mode == "none" and not args.one_sided:
                    nk = NcclKV(kv.plane, K)
                    nk.set_keys(keys)
                    back = torch.empty(len(keys), width, device=dev)

                    def nccl_pair():
                        nk.push(kt, vals)
                        nk.pull(kt, back)
                    before = pushes[0]
                    row["nccl_ms"] = round(timed(nccl_pair, args.iters), 4)
                    torch.cuda.synchronize()
                    n_all = before + 3 + args.iters
                    row["nccl_max_err"] = float((back - n_all * vals).abs().max().item() / n_all)
                    row["speedup_vs_nccl"] = round(row["nccl_ms"] / ms, 3)
                    kv.plane.check_status("nccl arm")
                out.append(row)
                if world > 1:
                    dist.barrier()
                if fab is not None:
                    fab.close()
                del kv
                torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps({"kernel": f"kv push+pull ({world} rank(s))", "results": out}))
    if world > 1:
        dist.destroy_process_group()


def bench_darlin(args):
    """Darlin passes on synthetic data (rows x 100 real-valued nonzeros, Zipf ids s=1.1,
    values |N(0,1)| normalised per row). One rank per GPU; with torch.distributed.run the
    (G, U) slices and the new weights travel over peer memory."""
    import time
    import numpy as np
    import torch.distributed as dist
    from ..models.darlin import DarlinConfig, DarlinRank, darlin_heap_bytes, run_darlin
    from ..parallel.fabric import Fabric
    from ..utils.synthetic import gen_batch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rows, z, nf = args.rows, args.z, 1 << args.log2_keys
    ids, y, vals = gen_batch(rows, z, nf, 1.1, seed=0, batch=rank, device=dev, ids64=True, real_values=True)
    from . import _lib as L
    keys = torch.empty_like(ids)
    L.check(L.lib().psb_hash_ids(0, L.ptr(ids), L.ptr(keys), ids.numel(), 40 << 56, L.stream_ptr()), "hash")
    cfg = DarlinConfig(lambda_l1=1.0, eta=0.9, block_cols=1 << 16, max_pass=args.passes, epsilon=0.0, tau=args.tau)
    hb = darlin_heap_bytes(cfg, world)
    fab = Fabric.from_process_group(hb) if world > 1 else Fabric.single(hb, dev)
    # global dictionary: all feature ids hashed (every rank can compute it without communication)
    allk = torch.empty(nf, dtype=torch.int64, device=dev)
    L.check(L.lib().psb_hash_ids(0, L.ptr(torch.arange(nf, dtype=torch.int64, device=dev)), L.ptr(allk), nf, 40 << 56,
                                 L.stream_ptr()), "hash")
    gk = torch.from_numpy(np.sort(allk.cpu().numpy().view(np.uint64)).view(np.int64)).to(dev)
    t0 = time.time()
    r = DarlinRank(fab, cfg, keys, y, fixed_z=z, vals=vals, global_keys=gk)
    torch.cuda.synchronize()
    prep = time.time() - t0

    def all_reduce(v, op):
        t = torch.tensor(v, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
        return t.tolist()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.time()
    if args.phases:
        r.phase_ns = torch.zeros(4, dtype=torch.int64, device=dev)
    hist = run_darlin([r], all_reduce=all_reduce if world > 1 else None, num_examples=rows * world)
    torch.cuda.synchronize()
    dt = time.time() - t0
    dev_ms = [h["device_ms"] for h in hist]
    if world > 1:
        t = torch.tensor(dev_ms, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms = t.tolist()
    if rank == 0:
        print(json.dumps({"kernel": "darlin", "gpus": world, "rows_per_gpu": rows, "nnz_per_row": z, "features": nf,
                          "blocks_per_pass": len(r.blocks), "tau": args.tau, "preprocess_s": prep,
                          "s_per_pass": dt / len(hist), "examples_per_s_per_pass": rows * world * len(hist) / dt,
                          "device_ms_per_pass_max_over_ranks": [round(v, 3) for v in dev_ms],
                          "examples_per_s_device": rows * world / (min(dev_ms) * 1e-3),
                          "phase_ms_per_pass_cta0": None if r.phase_ns is None else dict(zip(
                              ["load_parameter_blocks", "nonzero_passes", "barrier", "owner_update"],
                              [round(v / 1e6 / len(hist), 3) for v in r.phase_ns.tolist()])),
                          "objective": [h["objective"] for h in hist], "nnz_w": hist[-1]["nnz_w"]}))
    if world > 1:
        dist.barrier(); fab.close(); dist.destroy_process_group()


def bench_h2d(args):
    """Host-to-device copy ceiling of this box: every rank copies ``--mb`` MB from pinned host memory to
    its GPU ``--iters`` times in a row (two host buffers in turn, one stream), all ranks at the same
    time. GB/s per GPU from the slowest rank's CUDA-event time, and the sum over ranks: what an
    end-to-end training step that ships its minibatch from the host can reach at best."""
    dist, rank, world, dev = _dist_init()
    n = int(args.mb * 1000 * 1000)
    host = [torch.empty(n, dtype=torch.uint8).pin_memory() for _ in range(2)]
    for h in host:
        h.random_(0, 255)
    dst = [torch.empty(n, dtype=torch.uint8, device=dev) for _ in range(2)]
    st = torch.cuda.Stream(device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        for i in range(3):
            dst[i % 2].copy_(host[i % 2], non_blocking=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    with torch.cuda.stream(st):
        e0.record()
        for i in range(args.iters):
            dst[i % 2].copy_(host[i % 2], non_blocking=True)
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.iters
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({"kernel": "pinned host -> device copy", "gpus": world, "MB_per_copy": args.mb,
                          "ms_per_copy_max_over_ranks": round(ms, 4), "GB_per_s_per_gpu": n / (ms * 1e-3) / 1e9,
                          "GB_per_s_all_gpus": world * n / (ms * 1e-3) / 1e9}))
    if world > 1:
        dist.barrier(); dist.destroy_process_group()


def _dist_init():
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return dist, rank, world, dev


def _max_over_ranks(dist, world, dev, vals):
    t = torch.tensor(vals, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def bench_gather(args):
    """The random-access rate of this part at the table's density: n entries of 32 bytes picked from
    a table of 2^log2-slots entries, in address order (what a sorted key list with the order-preserving
    slot map produces) and in random order; a 16-byte load per entry (pull) and a read-modify-write
    (optimiser update). The roofline of the table walks of the pull and apply kernels is this rate,
    not the copy bandwidth."""
    from . import _lib
    from ._lib import check, ptr, stream_ptr
    dev = torch.device("cuda")
    L = _lib.lib()
    L.psb_probe_entries.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_int, C.c_void_p, C.c_void_p]
    cap, n = 1 << args.log2_slots, args.n
    table = torch.zeros(cap * 8, dtype=torch.float32, device=dev)
    flush = torch.empty(64 << 20, dtype=torch.int32, device=dev)
    out = torch.empty(n, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    rnd = torch.randint(0, cap, (n,), device=dev, generator=g, dtype=torch.int64).to(torch.int32)
    srt = torch.sort(rnd.to(torch.int64))[0].to(torch.int32)
    peak, tag = _peak_gbs()
    res = {"entries": n, "table_GB": cap * 32 / 1e9, "peak": tag}
    for order, idx in (("address_order", srt), ("random_order", rnd)):
        for mode, name, nbytes in ((0, "load16", 32), (1, "update", 64)):
            med, best = _time(lambda: check(L.psb_probe_entries(ptr(table), ptr(idx), n, mode, ptr(out), stream_ptr())),
                              args.iters, flush)
            res[f"{name}_{order}"] = {"ms": round(med, 4), "G_entries_per_s": round(n / 1e9 / (med * 1e-3), 2),
                                      "sector_GB_per_s": round(n * nbytes / 1e9 / (med * 1e-3), 1),
                                      "frac_of_copy_bw": round(n * nbytes / 1e9 / (med * 1e-3) / peak, 3)}
    print(json.dumps(res))


def bench_fabric(args):
    """Peer store and peer load bandwidth of this box, per direction and per GPU: every rank copies
    `--mb` MB to (store) and from (load) the heap of rank + d, for every distance d, with the same
    16-byte copy kernel the dense-layer path uses. The device counterpart of the reference's raw
    transport probe (test/network_perf_ps.cc:23-47); its result is the NVLink roofline to use.
    With one rank it measures the local copy."""
    from ..parameter.kv_layer import fabric_copy
    from ..parallel.fabric import Fabric
    dist, rank, world, dev = _dist_init()
    nbytes = args.mb << 20
    fab = Fabric.from_process_group(nbytes + 4096) if world > 1 else Fabric.single(nbytes + 4096, dev)
    local = torch.empty(nbytes // 4, dtype=torch.float32, device=dev).normal_()
    sink = torch.zeros(1, device=dev)
    res = {}
    for d in range(0 if world == 1 else 1, world):
        peer = (rank + d) % world
        for name, src, dst, mode in (("store", local.data_ptr(), fab.ptr(peer, 0), 0),
                                     ("load", fab.ptr(peer, 0), local.data_ptr(), 0),
                                     ("load_only", fab.ptr(peer, 0), local.data_ptr(), 1)):
            ts = []
            for i in range(args.iters + 2):
                if world > 1:
                    dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); fabric_copy(src, dst, nbytes, mode, sink); b.record()
                torch.cuda.synchronize()
                if i >= 2:
                    ts.append(a.elapsed_time(b))
            ts.sort()
            ms = _max_over_ranks(dist, world, dev, [ts[len(ts) // 2]])[0]
            res[f"{name}_d{d}"] = nbytes / 1e9 / (ms * 1e-3)
    if rank == 0:
        kinds = ("store", "load", "load_only")
        out = {"kernel": "fabric copy (16-byte peer accesses)", "gpus": world, "MB": args.mb,
               "GB_per_s_per_direction_per_gpu": {k: round(v, 1) for k, v in res.items()}}
        for k in kinds:
            v = [x for n, x in res.items() if n.startswith(k + "_d")]
            if v:
                out[f"{k}_min_over_distances"] = round(min(v), 1)
        print(json.dumps(out))
    if world > 1:
        dist.barrier(); fab.close(); dist.destroy_process_group()


def bench_layer(args):
    """Dense layers through DeviceKVLayer: for each layer of the reference's probe
    (AlexNet, test/kv_layer_perf_ps.cc:34-70) push + apply + pull, MB/s of layer data per worker
    as the reference prints, the achieved NVLink rate per GPU and direction, and NCCL
    reduce-scatter + all-gather of the same tensor for comparison. Max over ranks."""
    from ..parameter.kv_layer import DeviceKVLayer
    from ..parallel.fabric import Fabric
    dist, rank, world, dev = _dist_init()
    sizes = [11 * 11 * 96, 5 * 5 * 256, 3 * 3 * 284, 3 * 3 * 256, 43264 * 4096, 4096 * 4096, 4096 * 1000]
    if args.small:
        sizes = [s if s < (1 << 24) else s // 16 for s in sizes]
    layers = dict(enumerate(sizes))
    ring = 2
    fab = (Fabric.from_process_group(DeviceKVLayer.heap_bytes(layers, world, ring=ring)) if world > 1
           else Fabric.single(DeviceKVLayer.heap_bytes(layers, 1, ring=ring), dev))
    kv = DeviceKVLayer(fab, layers, updater="add", ring=ring)
    rows = []
    rounds = {lid: 0 for lid in layers}
    for lid, n in layers.items():
        data = torch.ones(n, device=dev)
        out = torch.empty(n, device=dev)
        ts, tn = [], []
        for i in range(args.iters + 2):
            if world > 1:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            kv.push(lid, data); kv.apply(lid); rounds[lid] += 1
            kv.pull(lid, out, wait_for_round=rounds[lid])
            b.record()
            torch.cuda.synchronize()
            if i >= 2:
                ts.append(a.elapsed_time(b))
            if world > 1 and n % world == 0:
                shard = torch.empty(n // world, device=dev)
                dist.barrier()
                a.record()
                dist.reduce_scatter_tensor(shard, data)
                dist.all_gather_into_tensor(out, shard)
                b.record()
                torch.cuda.synchronize()
                if i >= 2:
                    tn.append(a.elapsed_time(b))
        kv.check_status("layer bench")
        ts.sort(); tn.sort()
        ms = _max_over_ranks(dist, world, dev, [ts[len(ts) // 2]])[0]
        ms_n = _max_over_ranks(dist, world, dev, [tn[len(tn) // 2]])[0] if tn else None
        # Per direction and GPU: my push sends the (S-1)/S part of the layer out and the peers' pulls of my
        # shard send as much out again; the same two amounts come in (the peers' pushes, my pull).
        link = n * 4 * (world - 1) / max(1, world)
        rows.append({"layer": lid, "elements": n, "ms_push_apply_pull": round(ms, 4),
                     "MB_per_s_per_worker": round(n * 4 / 1e6 / (ms * 1e-3), 1),
                     "nvlink_GB_per_s_per_gpu_per_direction": round(2 * link / 1e9 / (ms * 1e-3), 1) if world > 1 else None,
                     "nccl_rs_ag_ms": None if ms_n is None else round(ms_n, 4)})
    if rank == 0:
        tot = sum(r["ms_push_apply_pull"] for r in rows)
        print(json.dumps({"kernel": "kv layer push + apply + pull", "gpus": world, "layers": rows,
                          "all_layers_MB_per_s_per_worker": round(sum(sizes) * 4 / 1e6 / (tot * 1e-3), 1)}))
    if world > 1:
        dist.barrier(); fab.close(); dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("sort"); s.add_argument("--n", type=int, default=65536 * 200)
    s.add_argument("--bits", type=int, default=64); s.add_argument("--iters", type=int, default=5)
    s = sub.add_parser("localize"); s.add_argument("--rows", type=int, default=65536); s.add_argument("--z", type=int, default=200)
    s.add_argument("--log2-keys", type=int, default=26); s.add_argument("--key-bits", type=int, default=40)
    s.add_argument("--method", default="auto", choices=["auto", "bucket", "sort"]); s.add_argument("--graph", action="store_true")
    s.add_argument("--iters", type=int, default=20); s.add_argument("--warmup", type=int, default=8)
    s = sub.add_parser("step"); s.add_argument("--rows", type=int, default=65536); s.add_argument("--z", type=int, default=200)
    s.add_argument("--log2-keys", type=int, default=26); s.add_argument("--iters", type=int, default=5)
    s.add_argument("--hashed-slots", action="store_true")
    s = sub.add_parser("wide"); s.add_argument("--rows", type=int, default=32768); s.add_argument("--z", type=int, default=40)
    s.add_argument("--log2-keys", type=int, default=22); s.add_argument("--n-ctx", type=int, default=128)
    s.add_argument("--iters", type=int, default=5)
    s = sub.add_parser("wide-step"); s.add_argument("--rows", type=int, default=32768); s.add_argument("--z", type=int, default=40)
    s.add_argument("--log2-keys", type=int, default=25); s.add_argument("--n-ctx", type=int, default=64)
    s.add_argument("--iters", type=int, default=20); s.add_argument("--tau", type=int, default=8); s.add_argument("--pool", type=int, default=4)
    s.add_argument("--one-sided", action="store_true", help="pull by remote probes instead of the exchange kernel")
    s.add_argument("--fused", action="store_true", help="add the products into the margins inside the pull kernel instead of storing P[U x N]")
    s = sub.add_parser("darlin"); s.add_argument("--phases", action="store_true"); s.add_argument("--rows", type=int, default=1250000); s.add_argument("--z", type=int, default=100)
    s.add_argument("--log2-keys", type=int, default=24); s.add_argument("--passes", type=int, default=3)
    s.add_argument("--tau", type=int, default=2)
    s = sub.add_parser("kv"); s.add_argument("--sizes", type=int, nargs="+", default=[1000, 100000, 1000000, 16000000])
    s.add_argument("--iters", type=int, default=5); s.add_argument("--quant", default="none", choices=["none", "int8", "fp16"])
    s.add_argument("--one-sided", action="store_true", help="pull with remote probes instead of the exchange kernel")
    s.add_argument("--widths", type=int, nargs="+", default=[1]); s.add_argument("--nccl", action="store_true")
    s.add_argument("--modes", nargs="+", default=["none"], choices=["none", "key_caching", "int8", "fp16"])
    s.add_argument("--max-values", type=int, default=1 << 26, help="skip K x width above this (memory of the inbox ring)")
    s = sub.add_parser("gather"); s.add_argument("--log2-slots", type=int, default=27)
    s.add_argument("--n", type=int, default=2680000); s.add_argument("--iters", type=int, default=5)
    s = sub.add_parser("h2d"); s.add_argument("--mb", type=float, default=52.7); s.add_argument("--iters", type=int, default=50)
    s = sub.add_parser("fabric"); s.add_argument("--mb", type=int, default=256); s.add_argument("--iters", type=int, default=5)
    s = sub.add_parser("layer"); s.add_argument("--iters", type=int, default=5)
    s.add_argument("--small", action="store_true", help="shrink the two largest layers 16x (quick runs)")
    args = ap.parse_args()
    import sys
    sys.path.insert(0, os.fspath(Path(__file__).resolve().parents[2]))
    from .. import _build
    _build.build_cuda()
    {"sort": bench_sort, "step": bench_step, "wide": bench_wide, "wide-step": bench_wide_step, "kv": bench_kv,
     "darlin": bench_darlin, "h2d": bench_h2d, "localize": bench_localize, "fabric": bench_fabric, "layer": bench_layer, "gather": bench_gather}[args.cmd](args)


if __name__ == "__main__":
    main()
