"""Multi-GPU self-tests of the planes that sit beside the sparse-LR path, over real peer
mappings (run under torch.distributed.run, one rank per GPU):

    --what layer    DeviceKVLayer: several rounds pushed back to back with no host barrier and
                    ranks of different speed (the inbox ring bounds the fast ones), against the CPU sum
    --what kv       DeviceKVMap (FTRL entries): collective push rounds and exchange pulls against
                    the CPU restatement of the table
    --what darlin   block coordinate descent over real peers against the NumPy restatement
    --what wide     wide values: the single cooperative launch with all three roles of the
                    exchange pull fused with the tcgen05 product, against fp32 PyTorch

Every wait in the kernels is bounded; nothing here injects a fault.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist


def _gather(obj):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def test_layer(rank, world, dev):
    from ..parameter.kv_layer import DeviceKVLayer
    from .fabric import Fabric
    layers = {0: 10, 1: 100_003, 2: 1 << 20, 5: 999}
    rounds, ring = 7, 2
    fab = Fabric.from_process_group(DeviceKVLayer.heap_bytes(layers, world, ring=ring))
    kv = DeviceKVLayer(fab, layers, partition_thr=1000, updater="add", ring=ring)
    streams = {lid: torch.cuda.Stream(device=dev) for lid in layers}       # layers on different streams

    def grad(r, rnd, lid, n):
        g = torch.arange(n, dtype=torch.float32, device=dev) % 13
        return (g + 1.0) * (r + 1) + rnd * 0.5 + lid

    dist.barrier()
    for rnd in range(rounds):
        if rank == rnd % world:
            time.sleep(0.02)                 # a different rank is slow in every round; nobody waits on the host
        for lid, n in layers.items():
            with torch.cuda.stream(streams[lid]):
                kv.push(lid, grad(rank, rnd, lid, n), stream=streams[lid])
                kv.apply(lid, stream=streams[lid])
    ok = True
    for lid, n in layers.items():
        out = torch.zeros(n, device=dev)
        with torch.cuda.stream(streams[lid]):
            kv.pull(lid, out, wait_for_round=rounds, stream=streams[lid])
        streams[lid].synchronize()
        exp = torch.zeros(n, device=dev)
        for rnd in range(rounds):
            for r in range(world):
                exp += grad(r, rnd, lid, n)
        if not torch.allclose(out, exp, rtol=1e-5, atol=1e-4):
            print(f"rank {rank} layer {lid}: max err {float((out - exp).abs().max())}")
            ok = False
    kv.check_status(f"rank {rank}")
    return ok, fab


def test_kv(rank, world, dev):
    from ..parameter.kv import DeviceKVMap
    from ..utils import oracle
    from .dataplane import OptimizerConfig
    opt = OptimizerConfig(algo="ftrl", alpha=0.1, beta=1.0, l1=0.01, l2=0.1)
    kv = DeviceKVMap.create(table_capacity=1 << 14, max_keys=1 << 12, opt=opt)
    rng = np.random.default_rng(7)              # the same stream on every rank: everybody knows everybody's data
    universe = np.unique(rng.integers(0, np.iinfo(np.uint64).max, 3000, dtype=np.uint64))
    ot = oracle.OracleTable(opt)
    rounds = 6
    for rnd in range(rounds):
        per = []
        for r in range(world):
            k = np.sort(rng.choice(universe, 400 if (rnd + r) % 3 else 0, replace=False))   # some ranks push nothing
            per.append((k, rng.normal(size=len(k)).astype(np.float32)))
        k, g = per[rank]
        kv.push(k, g)
        # the owner sums a round over the workers, then one entry update per key
        allk = np.unique(np.concatenate([p[0] for p in per])) if any(len(p[0]) for p in per) else np.zeros(0, np.uint64)
        gs = np.zeros(len(allk), np.float32)
        for pk, pg in per:
            gs[np.searchsorted(allk, pk)] += pg
        ot.push(allk, gs)
    mine = np.sort(rng.choice(universe, 1000, replace=False))[rank::world]
    ts = kv.pull(mine)
    kv.wait(ts)
    got = kv.result(ts).cpu().numpy()
    exp = ot.pull(mine)
    ok = bool(np.allclose(got, exp, rtol=2e-4, atol=2e-6))
    if not ok:
        print(f"rank {rank}: kv max err {np.abs(got - exp).max()}")
    return ok, kv.plane.fabric


def test_darlin(rank, world, dev):
    from ..models.darlin import DarlinConfig, DarlinRank, darlin_heap_bytes, run_darlin
    from ..utils import oracle
    from .fabric import Fabric
    rows, z, n_feat = 600, 10, 300
    cfg = DarlinConfig(lambda_l1=1.0, eta=0.9, block_cols=64, max_pass=4, epsilon=0.0, random_block_order=True,
                       kkt_ratio=10.0)
    rng = np.random.default_rng(100 + rank)
    ids = np.minimum((rng.pareto(1.1, rows * z) * 2).astype(np.int64), n_feat - 1)
    keys = oracle.hash_id_to_key(ids, 5)
    w_star = np.where(np.random.default_rng(1).random(n_feat) < 0.1, np.random.default_rng(2).normal(0, 2, n_feat), 0)
    y = np.where((w_star[ids]).reshape(rows, z).sum(1) + rng.logistic(size=rows) >= 0, 1.0, -1.0).astype(np.float32)
    parts = _gather((keys, y))
    gk = np.unique(np.concatenate([p[0] for p in parts]))
    fab = Fabric.from_process_group(darlin_heap_bytes(cfg, world))
    r = DarlinRank(fab, cfg, torch.from_numpy(keys.view(np.int64)).to(dev), torch.from_numpy(y).to(dev), fixed_z=z,
                   global_keys=torch.from_numpy(gk.view(np.int64)).to(dev))

    def all_reduce(vals, op):
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
        return t.tolist()

    hist = run_darlin([r], all_reduce=all_reduce, num_examples=rows * world)
    torch.cuda.synchronize()
    r.check_status(f"rank {rank}")
    models = _gather(r.my_model())
    ok = True
    if rank == 0:
        blocks = r.blocks
        orders = []
        for it in range(cfg.max_pass):
            o = list(range(len(blocks))); np.random.default_rng(1000 + it).shuffle(o)
            orders.append([blocks[i] for i in o])
        row_ptr = np.arange(rows + 1) * z
        w_ref, h_ref = oracle.darlin_oracle([(k, row_ptr, yy, None) for k, yy in parts], gk, cfg.lambda_l1, cfg.eta,
                                            cfg.delta_init, cfg.delta_max, orders, cfg.max_pass, cfg.kkt_ratio)
        got = np.zeros(len(gk), np.float32)
        for k, w in models:
            got[np.searchsorted(gk, k)] = w
        ok = bool(np.allclose([h["objective"] for h in hist], h_ref, rtol=2e-4)) and \
            bool(np.allclose(got, np.where(np.isnan(w_ref), 0, w_ref), rtol=2e-3, atol=2e-4))
        if not ok:
            print("darlin objective", [h["objective"] for h in hist], "oracle", h_ref)
    # With a block delay the pass kernel overlaps the blocks' steps across the GPUs: every wait must be
    # met (status 0) and the objectives must follow the delayed restatement. (Not to the last digit: on
    # the device the gradient of block i runs beside the margin update of block i - tau, so it sees
    # some of it.) A small step and many blocks, since a delay of tau blocks out of five diverges.
    import dataclasses
    for tau in (1, 2):
        cfg_t = dataclasses.replace(cfg, tau=tau, eta=0.3, block_cols=16, max_pass=5)
        fab_t = Fabric.from_process_group(darlin_heap_bytes(cfg_t, world))
        rt = DarlinRank(fab_t, cfg_t, torch.from_numpy(keys.view(np.int64)).to(dev), torch.from_numpy(y).to(dev), fixed_z=z,
                        global_keys=torch.from_numpy(gk.view(np.int64)).to(dev))
        ht = run_darlin([rt], all_reduce=all_reduce, num_examples=rows * world)
        torch.cuda.synchronize()
        rt.check_status(f"rank {rank} tau {tau}")
        if rank == 0:
            orders = []
            for it in range(cfg_t.max_pass):
                o = list(range(len(rt.blocks))); np.random.default_rng(1000 + it).shuffle(o)
                orders.append([rt.blocks[i] for i in o])
            _, h_ref = oracle.darlin_oracle([(k, row_ptr, yy, None) for k, yy in parts], gk, cfg_t.lambda_l1, cfg_t.eta,
                                            cfg_t.delta_init, cfg_t.delta_max, orders, cfg_t.max_pass, cfg_t.kkt_ratio, tau=tau)
            got = [h["objective"] for h in ht]
            if not (np.allclose(got, h_ref, rtol=5e-3) and got[-1] < got[0]):
                ok = False
                print(f"darlin with delay {tau}: objective", got, "delayed restatement", h_ref)
        dist.barrier()
        fab_t.close()
    return ok, fab


def test_wide(rank, world, dev):
    from ..ops.localize import LocalBatch
    from ..utils.oracle import hash_id_to_key
    from .fabric import Fabric
    from .wide import WideConfig, WidePlane, wide_layout
    rows, z, n_feat, N = 300, 12, 2500, 128
    cfg = WideConfig(table_capacity=1 << 13, inbox_cap=rows * z, ring=2, alpha=0.1, beta=1.0, pull_cap=rows * z)
    fab = Fabric.from_process_group(wide_layout(cfg, world).total())
    plane = WidePlane(fab, cfg)
    all_keys = hash_id_to_key(np.arange(n_feat), 11)
    g = torch.Generator().manual_seed(3)
    table = (torch.randn(n_feat, 64, generator=g) * 0.5).to(torch.bfloat16)
    known = np.random.default_rng(3).random(n_feat) < 0.8
    lo, hi = plane.bounds_host[rank], plane.bounds_host[rank + 1]
    sel = known & (all_keys >= np.uint64(lo)) & (all_keys < np.uint64(min(hi, (1 << 64) - 1)))
    plane.load(all_keys[sel], table[torch.from_numpy(sel)])
    rng = np.random.default_rng(50 + rank)
    ids = np.minimum((rng.pareto(1.2, rows * z) * 3).astype(np.int64), n_feat - 1).astype(np.int32)
    y = np.where(rng.random(rows) < 0.5, 1.0, -1.0).astype(np.float32)
    b = LocalBatch(rows, rows * z, world, dev)
    b.localize(torch.from_numpy(ids).to(dev), torch.from_numpy(y).to(dev), plane.bounds, fixed_z=z, hash_seed=11)
    ctx = (torch.randn(N, 64, generator=g) * 0.3).to(torch.bfloat16).to(dev)
    P = torch.zeros(rows * z, N, device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    ok = True
    for rnd in range(3):                       # both parities of the exchange buffers, and one reuse
        P.zero_()
        # one cooperative launch: requester, owner and product roles; the last round also adds the
        # products into the rows' margins (the fused form the training step uses)
        plane.pull_xgemm(b, ctx, P, rnd, fuse_margins=rnd == 2)
        if rnd == 2:
            plane.rowloss(b)                   # adds the keys with long segments, then loss and gcoef
        torch.cuda.synchronize()
        plane.check_status(f"rank {rank} round {rnd}")
        U = int(b.n_unique.item())
        uk = b.ukeys[:U].cpu().numpy().view(np.uint64)
        idx = np.searchsorted(all_keys[np.argsort(all_keys)], uk)
        order = np.argsort(all_keys)
        src = order[idx]
        Vref = torch.where(torch.from_numpy(known[src])[:, None], table[torch.from_numpy(src)].float(), torch.zeros(U, 64))
        if not torch.equal(plane.pulled_rows(rnd, U).cpu().float(), Vref):
            print(f"rank {rank} round {rnd}: pulled rows differ")
            ok = False
        Pref = Vref @ ctx.cpu().float().T
        if not torch.allclose(P[:U].cpu(), Pref, rtol=2e-3, atol=2e-3):
            print(f"rank {rank} round {rnd}: product max err {float((P[:U].cpu() - Pref).abs().max())}")
            ok = False
        if rnd == 2:
            col = b.csr_col[:rows * z].cpu().numpy().reshape(rows, z)
            mref = Pref[torch.from_numpy(col), torch.from_numpy(np.arange(rows) % N)[:, None]].sum(1)
            if not torch.allclose(b.margin[:rows].cpu(), mref, rtol=2e-3, atol=2e-3):
                print(f"rank {rank}: fused margins max err {float((b.margin[:rows].cpu() - mref).abs().max())}")
                ok = False
        dist.barrier()
    return ok, fab


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", required=True, choices=["layer", "kv", "darlin", "wide"])
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    ok, fab = {"layer": test_layer, "kv": test_kv, "darlin": test_darlin, "wide": test_wide}[args.what](rank, world, dev)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    fab.close()
    dist.destroy_process_group()
    if int(flag.item()) != 1:
        print("SELFTEST FAILED")
        sys.exit(1)
    if rank == 0:
        print("SELFTEST OK")


if __name__ == "__main__":
    main()
