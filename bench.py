#!/usr/bin/env python
"""Headline benchmark: FTRL-proximal sparse logistic regression through the
device parameter server (examples/s, whole job), plus push+pull keys/s.

Workload (synthetic, random-init): 2^26 hashed uint64 keys, rows with 200 binary
non-zeros (Zipf-like ids, s=1.05), 64k-row minibatch per worker, per-key fp32
(z, sqrt_n, w) state sharded by key range over the GPUs, bounded delay tau=4,
alpha 0.1, beta 1, l1 1, l2 0.1.

    python bench.py --gpus N --steps K --warmup W          (N=1: plain python;
    N>1: launched by torch.distributed.run, one rank per GPU)

Rank 0 prints one JSON line. ``value`` is timed on the device (CUDA events, max
over ranks) with the minibatches already resident in HBM; ``e2e`` runs the same
steps through ``SparseLRWorker.submit`` from pinned host memory and reads each
step's loss back to the host. The timed region of K steps is repeated
``--repeats`` times (each bracketed by barrier + synchronize); ``value`` is the
median repetition, ``ms_per_step_min/max`` the spread. With more than one GPU
the NCCL all-to-all-v arm (same local kernels, same pipelining) is measured in
the same invocation and reported as ``vs_nccl``; both arms report their
logloss after the same number of examples.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

PUBLISHED_FTRL_EXAMPLES_PER_S = 4.0e4   # online FTRL progress log of the reference (docker guide), derived


def reference_arm():
    if int(os.environ.get("RANK", "0")) != 0:          # under torch.distributed.run: one line, from rank 0
        return 0
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is a Makefile C++ project (no setup.py/pyproject; pip install fails) and its "
                       "build needs zeromq, protobuf+protoc, glog, gflags, snappy, Eigen3: none present offline",
    }))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons DURING the timed region (read-only
    NVML queries every 10 ms on a thread; nvidia-smi polling as a fallback)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.idx, self.sm, self.reasons, self.max_mhz = gpu_index, [], set(), None
        self.stop_flag = threading.Event()
        self.thread = None
        self.power = []

    def _loop(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            while not self.stop_flag.is_set():
                self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                try:
                    r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    r = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
                try:
                    self.power.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                except Exception:
                    pass
                time.sleep(0.01)
        except Exception as e:  # NVML unavailable: one nvidia-smi sample
            try:
                out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits",
                                      "-i", str(self.idx)], capture_output=True, text=True, timeout=10).stdout
                a = [float(x) for x in out.strip().split(",")]
                self.sm.append(a[0]); self.max_mhz = a[1]
            except Exception:
                self.reasons.add(f"clock sampling unavailable: {type(e).__name__}")

    def start(self):
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()
        time.sleep(0.05)     # let the first samples land before the timed region starts

    def stop(self):
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=5)
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(sm), "power_w_max": max(self.power) if self.power else None}


def gpu_numa_cpus(local_rank: int, sysfs: str = "/sys"):
    """(node, cpu set) of the NUMA node the GPU hangs off, or None when the machine does not say."""
    import torch
    pr = torch.cuda.get_device_properties(local_rank)
    bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
    return numa_cpus_of_pci_device(bdf, sysfs)


def numa_cpus_of_pci_device(bdf: str, sysfs: str = "/sys"):
    try:
        with open(f"{sysfs}/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read())
        if node < 0:
            return None
        with open(f"{sysfs}/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
    except (OSError, ValueError):
        return None
    cpus = set()
    for part in text.split(","):
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return node, cpus


def _bind_to_gpu_numa_node(local_rank: int):
    """Run this rank (and allocate its pinned staging buffers) on the CPU socket next to its GPU:
    with eight ranks copying tens of MB per step each, host buffers that all sit on one socket make the
    end-to-end rate depend on that socket's memory and on the link between the sockets. Only the
    process's CPU affinity changes; nothing of the GPU. Returns the node, or None if unknown."""
    found = gpu_numa_cpus(local_rank)
    if found is None:
        return None
    node, cpus = found
    allowed = cpus & os.sched_getaffinity(0)
    if len(allowed) < 2:
        return None
    try:
        os.sched_setaffinity(0, allowed)
    except OSError:
        return None
    return node


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl"])
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--nnz-per-row", type=int, default=200)
    ap.add_argument("--log2-keys", type=int, default=26)
    ap.add_argument("--tau", type=int, default=4)
    ap.add_argument("--pool", type=int, default=4, help="distinct minibatches cycled through")
    ap.add_argument("--quant", default="none")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-pack-ids", action="store_true", help="end-to-end arms: ship the ids as int32 instead of a bit stream")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--no-nccl-arm", action="store_true", help="skip the NCCL all-to-all-v arm (measured by default on >1 GPU)")
    ap.add_argument("--breakdown", action="store_true",
                    help="also time each stage (localise / pull+margins / push / apply) with CUDA events, "
                         "stages run back to back on one stream")
    ap.add_argument("--key-cache", action="store_true", help="enable the key-caching filter")
    ap.add_argument("--key-bits", type=int, default=40,
                    help="significant bits of the hashed uint64 keys (top bits); 64 = full-width keys. The radix "
                         "sort skips digit positions that are constant across the batch")
    ap.add_argument("--pull", default="exchange", choices=["exchange", "one-sided"],
                    help="exchange: keys to owners + weights back as bulk peer stores; one-sided: remote table probes")
    ap.add_argument("--hashed-slots", action="store_true",
                    help="re-hash keys into table slots instead of the order-preserving slot map")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_node = _bind_to_gpu_numa_node(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import __graft_entry__ as ge
    if rank == 0:
        ge.build()
    if world > 1:
        dist.barrier()

    from parameter_server_b200.models.sparse_lr import SparseLRConfig, SparseLRWorker
    from parameter_server_b200.ops import _lib
    from parameter_server_b200.parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig, heap_layout
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.utils.synthetic import gen_batch

    rows, z = args.rows, args.nnz_per_row
    nnz = rows * z
    n_feat = 1 << args.log2_keys
    cap = 1
    while cap < 2 * n_feat // world:
        cap *= 2
    inbox_cap = nnz if world == 1 else (nnz // world) * 5 // 4 + 4096
    pc = PlaneConfig(table_capacity=cap, inbox_cap=inbox_cap, ring=args.tau + 2, quant=args.quant,
                     ordered_slots=not args.hashed_slots, key_cache=args.key_cache,
                     pull_cap=nnz if (args.pull == "exchange" and args.impl == "ours") else 0)
    opt = OptimizerConfig(algo="ftrl", alpha=0.1, beta=1.0, l1=1.0, l2=0.1)
    hb = heap_layout(pc, world).total()
    fab = Fabric.from_process_group(hb) if world > 1 else Fabric.single(hb, dev)
    plane = DataPlane(fab, pc, opt)
    worker = SparseLRWorker(plane, SparseLRConfig(max_rows=rows, max_nnz=nnz, tau=args.tau, hash_seed=0,
                                                  hash_bits=args.key_bits % 64, pipeline=3))
    # pool of distinct minibatches (per rank different data): on device and in pinned host memory
    pool_d = [gen_batch(rows, z, n_feat, 1.05, seed=0, batch=rank * 100003 + i, device=dev)[:2]
              for i in range(args.pool)]
    # The end-to-end arms take their minibatches from pinned host memory as a loader would hand them over:
    # the loader knows the number of features, so it ships the ids as a bit stream of ceil(log2(features))
    # bits each (26 instead of 32 here) and the device unpacks them; --no-pack-ids keeps plain int32 ids.
    from parameter_server_b200.utils.idpack import PackedIds, bits_for
    pool_h = []
    id_bits = bits_for(n_feat - 1) if not args.no_pack_ids else 32
    if not args.no_e2e:
        for ids, y in pool_d:
            ids_h = PackedIds.from_ids(ids, id_bits) if id_bits < 32 else ids.cpu().pin_memory()
            pool_h.append((ids_h, y.cpu().pin_memory()))
    torch.cuda.synchronize()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    nccl = None
    want_nccl = world > 1 and (args.impl == "nccl" or not args.no_nccl_arm)
    if args.impl == "nccl":
        assert world > 1, "--impl nccl needs at least two ranks"

    def run(pool, n, log=None):
        for i in range(n):
            ids, y = pool[i % len(pool)]
            worker.submit(ids, y, fixed_z=z)
            if log is not None:
                # D2H read of this step's running loss/accuracy counters (async, pinned)
                with torch.cuda.stream(worker.main_stream):
                    log[i].copy_(plane.pull_stats, non_blocking=True)
        worker.wait()

    def run_nccl(pool, n, log=None):
        """The baseline arm with the same overlap as the fused one: minibatch i+1 is copied and localised
        (and its split sizes exchanged) on the prep stream while minibatch i goes through NCCL push/pull."""
        prep, main_s = worker.prep_stream, worker.main_stream
        cur = torch.cuda.current_stream()
        prep.wait_stream(cur); main_s.wait_stream(cur)
        evs = [torch.cuda.Event(), torch.cuda.Event()]
        free = [torch.cuda.Event(), torch.cuda.Event()]
        for i in range(n + 1):
            if i < n:
                k = i % 2
                ids, y = pool[i % len(pool)]
                with torch.cuda.stream(prep):
                    if i >= 2:
                        prep.wait_event(free[k])
                    if isinstance(ids, PackedIds):
                        ids_d = ids if ids.is_cuda else PackedIds(ids.words.to(dev, non_blocking=True), ids.bits, ids.n)
                    else:
                        ids_d = ids if ids.is_cuda else ids.to(dev, non_blocking=True)
                    y_d = y if y.is_cuda else y.to(dev, non_blocking=True)
                    worker.bufs[k].localize(ids_d, y_d, plane.bounds, fixed_z=z, hash_seed=0,
                                            hash_bits=args.key_bits % 64, stream=prep)
                    nccl.exchange_counts(worker.bufs[k], k)
                    evs[k].record(prep)
            if i >= 1:
                k = (i - 1) % 2
                with torch.cuda.stream(main_s):
                    main_s.wait_event(evs[k])
                    nccl.step(worker.bufs[k], worker.step_no, counts_slot=k)
                    free[k].record(main_s)
                    worker.step_no += 1
                    if log is not None:
                        log[i - 1].copy_(plane.pull_stats, non_blocking=True)
        cur.wait_stream(main_s); cur.wait_stream(prep)

    def timed(fn, pool):
        """`repeats` regions of exactly `steps` steps, each between barrier + synchronize; device time, max over ranks."""
        out = []
        for _ in range(max(1, args.repeats)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sync_all()
            e0.record()
            fn(pool, args.steps)
            e1.record()
            sync_all()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out.append(float(t.item()))
        return sorted(out)

    def timed_e2e(fn, pool_host):
        log = torch.zeros((args.steps, 4), dtype=torch.float64).pin_memory()
        fn(pool_host, 7)        # untimed: every staging buffer has been through its graph capture afterwards
        out = []
        for _ in range(max(1, min(args.repeats, 3))):
            sync_all()
            t0 = time.perf_counter()
            fn(pool_host, args.steps, log)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            sync_all()
            tt = torch.tensor([t1 - t0], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            out.append(float(tt.item()))
        out.sort()
        return out[len(out) // 2], log

    def examples_and_loss():
        p = worker.read_progress()
        t = torch.tensor([p["loss_sum"], p["n_examples"]], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t)
        return float(t[1].item()), float(t[0].item()) / max(1.0, float(t[1].item()))

    # ---------------- NCCL arm first (its own table: the two arms must not train each other's model)
    nccl_res = None
    if want_nccl:
        from parameter_server_b200.parallel.nccl_baseline import NcclPushPull
        pc_n = PlaneConfig(table_capacity=cap, inbox_cap=16, ring=args.tau + 2, quant="none",
                           ordered_slots=not args.hashed_slots, pull_cap=0)
        fab_n = Fabric.from_process_group(heap_layout(pc_n, world).total())
        plane_f, worker_f = plane, worker
        plane = DataPlane(fab_n, pc_n, opt)
        worker = SparseLRWorker(plane, SparseLRConfig(max_rows=rows, max_nnz=nnz, tau=args.tau, hash_seed=0,
                                                      hash_bits=args.key_bits % 64, pipeline=3))
        nccl = NcclPushPull(plane, nnz)
        run_nccl(pool_d, args.warmup)
        sync_all()
        plane.check_status("nccl warm-up")
        worker.read_progress()
        ts_n = timed(run_nccl, pool_d)
        n_ex, n_loss = examples_and_loss()
        e2e_n = None
        if not args.no_e2e:
            sec, _ = timed_e2e(run_nccl, pool_h)
            e2e_n = world * rows * args.steps / sec
        plane.check_status("nccl arm")
        med = ts_n[len(ts_n) // 2]
        nccl_res = {"ms_per_step": med / args.steps, "examples_per_s": world * rows * args.steps / (med * 1e-3),
                    "e2e_examples_per_s": e2e_n, "logloss": n_loss, "after_examples": n_ex,
                    "collectives_per_step": 4}
        if args.impl == "nccl":
            ts, launches = ts_n, 0
        fab_n.close()
        del nccl
        nccl = None
        plane, worker = plane_f, worker_f

    # ---------------- device-timed arm
    uniq, clocks, e2e, ours_loss = [0], None, None, None
    if args.impl != "nccl":
        run(pool_d, args.warmup)
        sync_all()
        plane.check_status("warm-up")
        worker.read_progress()
        uniq = [int(b.n_unique.item()) for b in worker.bufs]
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        l0 = _lib.LAUNCHES
        ts = timed(run, pool_d)
        launches = (_lib.LAUNCHES - l0) // max(1, args.repeats)
        clocks = sampler.stop() if rank == 0 else None
        plane.check_status("timed region")
        ours_ex, ours_loss = examples_and_loss()
        # ---------------- end-to-end arm (pinned host inputs, per-step D2H of the loss counters)
        if not args.no_e2e:
            sec, log = timed_e2e(run, pool_h)
            plane.check_status("e2e region")
            h2d = (pool_h[0][0].nbytes() if isinstance(pool_h[0][0], PackedIds) else nnz * 4) + rows * 4
            e2e = {"value": world * rows * args.steps / sec, "unit": "examples/s",
                   "h2d_bytes_per_step": world * h2d, "d2h_bytes_per_step": world * 32,
                   "h2d_GB_per_s_per_gpu": h2d * args.steps / sec / 1e9,
                   "loss_per_example_last": float((log[-1, 0] - log[-2, 0]) / max(1.0, float(log[-1, 2] - log[-2, 2])))
                   if args.steps > 1 else None}
    ms = ts[len(ts) // 2]
    ex_per_s = world * rows * args.steps / (ms * 1e-3)

    breakdown = None
    if args.breakdown and args.impl != "nccl":
        names = ["localize", "pull_margin", "push", "apply"]
        acc = {k: 0.0 for k in names}
        reps = 6
        for i in range(reps + 2):
            ids, y = pool_d[i % len(pool_d)]
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
            sync_all()
            ev[0].record()
            b = worker.prepare(ids, y, fixed_z=z)
            ev[1].record()
            t_ = worker.step_no
            if pc.pull_cap:
                plane.pull_exchange(b, t_, need_applied=max(0, t_ - args.tau))
            else:
                plane.pull_margin(b, need_applied=max(0, t_ - args.tau))
            ev[2].record()
            plane.push(b, t_, send_keys=not pc.pull_cap)
            ev[3].record()
            plane.apply(t_)
            ev[4].record()
            worker.step_no += 1
            torch.cuda.synchronize()
            if i >= 2:
                for k, name in enumerate(names):
                    acc[name] += ev[k].elapsed_time(ev[k + 1]) / reps
        sync_all()
        tb = torch.tensor([acc[k] for k in names], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tb, op=dist.ReduceOp.MAX)
        breakdown = {k: float(v) for k, v in zip(names, tb.tolist())}
        plane.check_status("breakdown")

    if rank == 0:
        u_mean = sum(uniq) / len(uniq)
        out = {
            "metric": "FTRL sparse-LR examples/sec (whole job); push+pull keys/sec in config",
            "value": ex_per_s, "unit": "examples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "repeats": len(ts), "ms_per_step_min": ts[0] / args.steps, "ms_per_step_max": ts[-1] / args.steps,
            "scaling": "weak", "vs_baseline": ex_per_s / PUBLISHED_FTRL_EXAMPLES_PER_S,
            "dtype": "fp32", "data": "synthetic (device generator, Zipf-like ids, random-init model)",
            "impl": args.impl,
            "config": {"model": "FTRL-proximal L1/L2 logistic regression", "global_batch": world * rows,
                       "rows_per_worker": rows, "nnz_per_row": z, "keys": f"2^{args.log2_keys} ids hashed on the device to uint64 keys "
                                                        f"({args.key_bits} significant bits, in the top bits)",
                       "seq_len": z, "parallelism": f"dp{world} x key-range shards{world}", "tau": args.tau,
                       "alpha": 0.1, "beta": 1.0, "l1": 1.0, "l2": 0.1, "quant": args.quant, "ordered_slots": not args.hashed_slots, "pull": args.pull,
                       "unique_keys_per_step_per_worker": u_mean,
                       "push_pull_keys_per_s": 2 * u_mean * world * args.steps / (ms * 1e-3),
                       "host_numa_node": numa_node,
                       "e2e_input": (f"ids as a {id_bits}-bit stream from pinned host memory, unpacked on the device" if id_bits < 32
                                     else "int32 ids from pinned host memory"),
                       "l2_policy": f"inputs larger than L2: {args.pool} distinct minibatches of "
                                    f"{nnz * 4 / 1e6:.0f} MB ids, >=300 MB sort working set per step"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "stage_ms_max_over_ranks": breakdown,
            "logloss_after_examples": None if ours_loss is None else {"examples": ours_ex, "logloss": ours_loss},
            "nccl_arm": nccl_res,
            "vs_nccl": None if (nccl_res is None or args.impl == "nccl") else {
                "device_timed": ex_per_s / nccl_res["examples_per_s"],
                "e2e": (e2e["value"] / nccl_res["e2e_examples_per_s"]) if (e2e and nccl_res["e2e_examples_per_s"]) else None},
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        fab.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
