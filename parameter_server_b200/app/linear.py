"""Linear methods on the GPUs, configured by the reference's text format.

    python -m parameter_server_b200.app.linear -app_file online_l1lr.conf            # one GPU
    python -m torch.distributed.run --nproc-per-node 8 -m parameter_server_b200.app.linear -app_file x.conf

Accepts the ``PS.LM.Config`` text format (``app/linear_method/proto/linear.proto:7-101``):
``async_sgd { ... }`` trains FTRL-proximal / AdaGrad / SGD through the device
parameter server (one shard + one worker per GPU), ``darlin { ... }`` runs block
coordinate descent, and a configuration with only ``validation_data`` +
``model_input`` evaluates a saved model. The model is written as one text file
per shard, ``<model_output.file>_S<rank>``, one ``key<TAB>weight`` line per
non-zero weight, which is what the reference's servers write
(``parameter/kv_map.h:100-117``) and what its evaluator reads back.
"""
from __future__ import annotations

import argparse
import glob
import os
import sys
import time
from typing import List, Optional

import numpy as np
import torch

from ..system import core


def _files(conf_data) -> List[str]:
    pats = conf_data.get("file", [])
    pats = pats if isinstance(pats, list) else [pats]
    hdfs = conf_data.get("hdfs")          # data { hdfs { home ugi namenode } }: the files are read through `hadoop fs`
    # format BIN: a matrix x is a handful of files (x.index, x.offset, x.label, x.info, ...); the search returns x
    return list(core.search_files(pats, hdfs if isinstance(hdfs, dict) else None, conf_data.get("format", "TEXT")))


def _penalty(conf):
    p = conf.get("penalty", {})
    lam = p.get("lambda", ["0"])
    lam = lam if isinstance(lam, list) else [lam]
    lam = [float(x) for x in lam]
    if p.get("type", "L1") == "L2":
        return 0.0, lam[0]
    return lam[0], (lam[1] if len(lam) > 1 else 0.0)


def _dist():
    import torch.distributed as dist
    if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        if not dist.is_initialized():
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        return dist, dist.get_rank(), dist.get_world_size()
    return None, 0, 1


def format_weight(v: float) -> str:
    """Default iostream formatting of a float: 6 significant digits."""
    return "%g" % v


def write_model(path: str, keys, weights):
    with open(path, "w") as out:
        for k, v in zip(keys.tolist(), weights.tolist()):
            out.write(f"{k}\t{format_weight(v)}\n")


class GpuEngine:
    """The device side of one rank for the node layer (``app/nodes.py``): a lock-step round is one
    ``SparseLRWorker.submit`` from pinned host buffers; nothing here waits for the device except the
    progress read-out and the end of the job."""

    def __init__(self, worker, plane, max_rows: int, max_nnz: int, real_values: bool, depth: int = 4):
        self.worker, self.plane = worker, plane
        self.ring = []
        for _ in range(depth):
            self.ring.append({
                "ids": torch.empty(max_nnz, dtype=torch.int64).pin_memory(),
                "vals": torch.empty(max_nnz, dtype=torch.float32).pin_memory() if real_values else None,
                "rp": torch.empty(max_rows + 1, dtype=torch.int32).pin_memory(),
                "y": torch.empty(max_rows, dtype=torch.float32).pin_memory(),
                "ev": torch.cuda.Event(),
                "used": False,
            })
        self.k = 0
        self.real_values = real_values

    def submit(self, batch) -> int:
        slot = self.ring[self.k % len(self.ring)]
        self.k += 1
        if slot["used"]:
            slot["ev"].synchronize()          # the copy that last read this pinned buffer is long done
        if batch is None:
            n, nnz = 0, 0
            slot["rp"][0] = 0
            vals = None
        else:
            yv, mats = batch
            m = mats[0]
            n, nnz = len(yv), m["index"].size
            slot["ids"][:nnz].copy_(torch.from_numpy(m["index"].view(np.int64)))
            slot["rp"][:n + 1].copy_(torch.from_numpy(m["offset"].astype(np.int32)))
            slot["y"][:n].copy_(torch.from_numpy(np.where(yv > 0, 1.0, -1.0).astype(np.float32)))
            vals = None
            if self.real_values:
                vals = slot["vals"][:nnz]
                if m["binary"]:
                    vals.fill_(1.0)
                else:
                    vals.copy_(torch.from_numpy(m["value"]))
        rows = n
        if nnz == 0 and n > 0:
            # every nonzero of the minibatch was filtered out (tail features): the round runs empty, as when
            # there is no minibatch; the rows still count as read
            n = 0
            slot["rp"][0] = 0
            vals = None
        self.worker.submit(slot["ids"][:nnz], slot["y"][:n], row_ptr=slot["rp"][:n + 1], vals=vals)
        slot["ev"].record(self.worker.copy_stream)
        slot["used"] = True
        return rows

    def finish(self):
        self.worker.wait()
        torch.cuda.synchronize()
        self.plane.check_status("async sgd")

    def progress(self) -> dict:
        p = self.worker.read_progress()
        if self.worker.auc_hist is not None:
            p["auc"] = auc_from_histogram(self.worker.auc_hist.cpu().numpy())
            self.worker.auc_hist.zero_()
        return p

    def set_alive(self, rank: int, alive: bool):
        self.plane.set_alive(rank, alive)

    def save_model(self, path: str):
        keys, w = self.plane.dump_nonzero()
        write_model(path, keys.numpy(), w.numpy())


def _scheduler_address(dist, rank: int, world: int) -> tuple:
    """The scheduler node's address for this job: ``PSB_SCHEDULER`` if given, else rank 0 picks a free
    port and publishes it through the launcher's key-value store; a single process uses the
    in-process van. Returns ``(spec, inproc)``."""
    from . import nodes
    from ..system import core as _core
    if os.environ.get("PSB_SCHEDULER"):
        return os.environ["PSB_SCHEDULER"], False
    if dist is None or world == 1:
        return nodes.scheduler_spec("inproc", 20000 + (os.getpid() % 20000)), True
    store = dist.distributed_c10d._get_default_store()
    if rank == 0:
        spec = nodes.scheduler_spec("127.0.0.1", _core.free_port())
        store.set("psb/scheduler", spec)
        return spec, False
    return store.get("psb/scheduler").decode(), False


def run_async_sgd(conf, verbose=True, engine: str = "gpu"):
    """Asynchronous SGD (FTRL / AdaGrad / SGD) with every rank a server node plus a worker node of the
    host control plane (``app/nodes.py``): files come from the scheduler's workload pool, progress
    goes to its monitor, the model dump is its ``SAVE_MODEL`` task, lost nodes are learned from the
    manager. ``engine="null"`` runs the same control flow without a device (tests)."""
    from . import nodes

    sgd = conf["async_sgd"]
    minibatch = int(sgd.get("minibatch", 1000))
    tau = int(sgd.get("max_delay", 0))
    passes = int(sgd.get("num_data_pass", 1))
    data = conf["training_data"]
    files = _files(data)
    text = data.get("text", "LIBSVM")
    fmt = data.get("format", "TEXT")
    out = conf.get("model_output", {}).get("file")
    if out:
        out = out if isinstance(out, str) else out[0]

    if engine == "null":
        dist, rank, world = None, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        eng = nodes.NullEngine(float(os.environ.get("PSB_NULL_STEP_SECONDS", "0")))
        fab = plane = None
    else:
        from ..models.sparse_lr import SparseLRConfig, SparseLRWorker
        from ..parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig, heap_layout
        from ..parallel.fabric import Fabric
        dist, rank, world = _dist()
        dev = torch.device("cuda", torch.cuda.current_device())
        l1, l2 = _penalty(conf)
        lr = conf.get("learning_rate", {})
        algo = "ftrl" if sgd.get("algo", "FTRL") == "FTRL" else ("adagrad" if sgd.get("ada_grad", "true") == "true" else "sgd")
        opt = OptimizerConfig(algo=algo, alpha=float(lr.get("alpha", 1)), beta=float(lr.get("beta", 1)), l1=l1, l2=l2,
                              lr_type="constant" if lr.get("type", "DECAY") == "CONSTANT" else "decay")
        def _filter_list(name):
            v = sgd.get(name, [])
            return v if isinstance(v, list) else [v]

        quant = "none"
        key_cache = False
        for name in ("push_filter", "pull_filter"):
            for f in _filter_list(name):
                kind = f.get("type")
                if kind == "FIXING_FLOAT" and name == "push_filter":
                    quant = "int8" if int(f.get("num_bytes", 3)) <= 1 else "fp16"
                elif kind == "KEY_CACHING":
                    key_cache = True          # one switch: repeated key lists skip the keys (push) and the probes (pull)
                elif rank == 0 and verbose:
                    # pulled weights travel as fp32, nothing is compressed on NVLink, and the gradient never
                    # leaves the fused kernel between its computation and the push: these have no place here
                    print(f"note: {name} {kind} is not applied by the GPU application", flush=True)
        max_nnz = int(os.environ.get("PSB_MAX_NNZ_PER_ROW", "512")) * minibatch
        table_cap = 1 << int(os.environ.get("PSB_LOG2_TABLE", "22"))
        # two-sided exchange pull; the key-caching filter, when asked for, is decided inside that kernel
        pc = PlaneConfig(table_capacity=table_cap, inbox_cap=max_nnz, ring=tau + 2, quant=quant, key_cache=key_cache,
                         ordered_slots=os.environ.get("PSB_ORDERED_SLOTS", "0") == "1", pull_cap=max_nnz)
        hb = heap_layout(pc, world).total()
        fab = Fabric.from_process_group(hb) if world > 1 else Fabric.single(hb, dev)
        plane = DataPlane(fab, pc, opt)
        if conf.get("_checkpoint_in"):
            from ..utils import checkpoint
            checkpoint.load_plane(plane, conf["_checkpoint_in"])
        real_values = text not in ("SPARSE_BINARY", "ADFEA", "TERAFEA", "CRITEO")
        worker = SparseLRWorker(plane, SparseLRConfig(max_rows=minibatch, max_nnz=max_nnz, tau=tau, hash_seed=None,
                                                      pipeline=2, auc=True, real_values=real_values))
        eng = GpuEngine(worker, plane, minibatch, max_nnz, real_values)

    lost = []

    def on_node_lost(node_id: str):
        # REMOVE_NODE from the manager: the dead rank's rounds are not waited for any more
        r = nodes.node_rank(node_id)
        lost.append(node_id)
        if r is not None and r != rank:
            eng.set_alive(r, False)
        if verbose:
            print(f"[rank {rank}] node {node_id} lost", flush=True)

    spec, inproc = _scheduler_address(dist, rank, world)
    rn = nodes.start_rank_nodes(rank, world, spec, files=files, data_format=fmt, text=text, passes=passes,
                                lease=int(os.environ.get("PSB_ROUND_LEASE", "64")),
                                roles=os.environ.get("PSB_ROLES", "HSW"), on_node_lost=on_node_lost, inproc=inproc)
    res = nodes.run_lockstep_worker_loop(rn, eng, minibatch=minibatch, data_format=fmt, text=text,
                                         report_interval=float(sgd.get("report_interval", 1)), model_file=out,
                                         announce=f"[rank {rank}]" if verbose else "",
                                         tail_filter=nodes.TailFeatureFilter(int(sgd["tail_feature_freq"]),
                                                                             float(sgd.get("countmin_n", 1e8)),
                                                                             int(sgd.get("countmin_k", 2)))
                                         if int(sgd.get("tail_feature_freq", 0)) > 0 else None)
    if conf.get("_checkpoint_out") and plane is not None:
        from ..utils import checkpoint
        checkpoint.save_plane(plane, conf["_checkpoint_out"], meta={"minibatches": res["rounds"], "examples": res["examples"]})
    if verbose:
        print(f"[rank {rank}] rounds {res['rounds']} examples {res['examples']} files {res['files']} lost {lost}", flush=True)
    if dist is not None:
        dist.barrier()
        fab.close()
    return dict(steps=res["rounds"], examples=res["examples"], files=res["files"], lost=lost)


def auc_from_histogram(h: np.ndarray) -> float:
    """AUC from the [2][4096] histogram of sigmoid(margin) by label."""
    neg, pos = h[:4096].astype(np.float64), h[4096:].astype(np.float64)
    if pos.sum() == 0 or neg.sum() == 0:
        return 0.5
    cum_neg = np.concatenate([[0], np.cumsum(neg)[:-1]])
    return float((pos * (cum_neg + neg / 2)).sum() / (pos.sum() * neg.sum()))


def run_evaluation(conf, verbose=True):
    """Model evaluation on one GPU (``app/linear_method/model_evaluation.h:27-107``):
    load ``key value`` files into a device table, stream the validation data,
    margins by table lookup, AUC / accuracy / logloss."""
    from ..models.sparse_lr import SparseLRConfig, SparseLRWorker
    from ..parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig, heap_layout
    from ..parallel.fabric import Fabric

    dev = torch.device("cuda", torch.cuda.current_device())
    model_files = _files(conf["model_input"])
    ks, ws = [], []
    for f in model_files:
        for line in open(f):
            a = line.split()
            if len(a) == 2:
                ks.append(int(a[0])); ws.append(float(a[1]))
    keys = np.array(ks, dtype=np.uint64)
    cap = 1 << max(12, int(np.ceil(np.log2(max(2, 2 * len(keys))))))
    chunk = 100000
    max_nnz = int(os.environ.get("PSB_MAX_NNZ_PER_ROW", "512")) * chunk
    pc = PlaneConfig(table_capacity=cap, inbox_cap=16, ring=2)
    fab = Fabric.single(heap_layout(pc, 1).total(), dev)
    plane = DataPlane(fab, pc, OptimizerConfig())
    plane.load_state(keys, w=torch.tensor(ws, dtype=torch.float32))
    worker = SparseLRWorker(plane, SparseLRConfig(max_rows=chunk, max_nnz=max_nnz, hash_seed=None, pipeline=1, real_values=True))
    data = conf["validation_data"]
    reader = core.StreamReader(_files(data), data.get("format", "TEXT"), data.get("text", "LIBSVM"), True)
    ys, ms = [], []
    while True:
        got = reader.read_matrices(chunk)
        if got is None:
            break
        yv, mats = got
        if not mats:
            continue
        m = mats[0]
        b = worker.prepare(torch.from_numpy(m["index"].view(np.int64)).to(dev),
                           torch.from_numpy(np.where(yv > 0, 1.0, -1.0).astype(np.float32)).to(dev),
                           row_ptr=torch.from_numpy(m["offset"].astype(np.int32)).to(dev),
                           vals=None if m["binary"] else torch.from_numpy(m["value"]).to(dev))
        plane.pull_margin(b)
        torch.cuda.synchronize()
        ys.append(yv); ms.append(b.margin[:len(yv)].cpu().numpy())
    y, margin = np.concatenate(ys), np.concatenate(ms)
    ev = core.evaluate(y.astype(np.float32), margin.astype(np.float32))
    if verbose:
        print(f"load {len(keys)} model entries\nload {len(y)} examples")
        print(f"auc: {ev['auc']:.6f}\naccuracy: {ev['accuracy']:.6f}\nlogloss: {ev['logloss']:.6f}")
    return ev


def run_darlin(conf, verbose=True):
    """Darlin (block coordinate descent, L1 logistic regression) on the GPUs. Preprocessing runs on the
    device (``models/darlin_prep.py``): tail-feature filter through the count-min kernels, the global
    column space as a device union of the ranks' key sets, feature groups cut into
    ``ceil(nnz per row * feature_block_ratio)`` blocks, prior groups first; ``save_model_every_n_iter``
    writes intermediate models."""
    from ..models.darlin import DarlinConfig, DarlinRank, darlin_heap_bytes, run_darlin as drive
    from ..models.darlin_prep import build_columns, plan_blocks
    from ..parallel.fabric import Fabric
    from ..utils.range import Range

    dist, rank, world = _dist()
    dev = torch.device("cuda", torch.cuda.current_device())
    d = conf["darlin"]
    init_w = d.get("init_w", {})
    init_type = init_w.get("type", "ZERO") if isinstance(init_w, dict) else "ZERO"
    if init_type not in ("ZERO", "CONSTANT", "GAUSSIAN"):
        raise SystemExit(f"darlin.init_w type {init_type} is not supported by the GPU application: "
                         "run this configuration on the CPU nodes (bin/psb_linear)")
    l1, _ = _penalty(conf)
    data = conf["training_data"]
    files = _files(data)[rank::world]
    by_group = str(data.get("ignore_feature_group", "false")) != "true"
    reader = core.StreamReader(files, data.get("format", "TEXT"), data.get("text", "LIBSVM"), not by_group)
    groups = {}          # group id -> lists of chunks
    ys, n_rows = [], 0
    while True:
        got = reader.read_matrices(100000) if files else None
        if got is None:
            break
        yv, mats = got
        if not mats:
            continue
        for m in mats:
            g = groups.setdefault(int(m["id"]), dict(id=int(m["id"]), index=[], offset=[np.zeros(1, np.int64)], value=[],
                                                     binary=True, rows=0))
            # a group may be absent from earlier chunks: its rows there are empty
            if g["rows"] < n_rows:
                g["offset"].append(np.full(n_rows - g["rows"], g["offset"][-1][-1], np.int64))
            g["index"].append(m["index"])
            g["offset"].append(m["offset"][1:].astype(np.int64) + g["offset"][-1][-1])
            if not m["binary"]:
                g["binary"] = False
                g["value"].append(m["value"])
            elif not g["binary"]:
                g["value"].append(np.ones(len(m["index"]), np.float32))
            g["rows"] = n_rows + len(yv)
        ys.append(yv)
        n_rows += len(yv)
    glist = []
    for g in groups.values():
        if g["rows"] < n_rows:
            g["offset"].append(np.full(n_rows - g["rows"], g["offset"][-1][-1], np.int64))
        glist.append(dict(id=g["id"], index=np.concatenate(g["index"]) if g["index"] else np.zeros(0, np.uint64),
                          offset=np.concatenate(g["offset"]), binary=g["binary"],
                          value=np.concatenate(g["value"]) if g["value"] else np.zeros(0, np.float32)))
    if not glist:
        glist = [dict(id=0, index=np.zeros(0, np.uint64), offset=np.zeros(n_rows + 1, np.int64), binary=True,
                      value=np.zeros(0, np.float32))]
    y = np.where(np.concatenate(ys) > 0, 1.0, -1.0).astype(np.float32) if ys else np.zeros(0, np.float32)
    tail = int(d.get("tail_feature_freq", 0))
    nnz_local = sum(len(g["index"]) for g in glist)
    cells = int(min(1 << 28, max(1 << 16, float(d.get("countmin_n_ratio", 2.0)) * max(1, nnz_local) * world)))
    col, row_ptr, vals, space = build_columns(glist, n_rows, dev, dist=dist, tail_freq=tail, countmin_cells=cells,
                                              countmin_k=int(d.get("countmin_k", 2)))
    prior = d.get("prior_fea_group", [])
    prior = [int(x) for x in (prior if isinstance(prior, list) else [prior])]
    plan = plan_blocks(space, feature_block_ratio=float(d.get("feature_block_ratio", 4)),
                       max_block_cols=int(os.environ.get("PSB_DARLIN_BLOCK", str(1 << 16))), prior_groups=prior,
                       prior_iters=int(d.get("num_iter_for_prior_fea_group", 5)))
    cfg = DarlinConfig(lambda_l1=l1, eta=float(conf.get("learning_rate", {}).get("alpha", 1.0)),
                       delta_init=float(d.get("delta_init_value", 1)), delta_max=float(d.get("delta_max_value", 5)),
                       kkt_ratio=float(d.get("kkt_filter_threshold_ratio", 10)), max_pass=int(d.get("max_pass_of_data", 10)),
                       epsilon=float(d.get("epsilon", 1e-4)), tau=int(d.get("max_block_delay", 0)),
                       block_cols=max(1, plan.block_cols),
                       random_block_order=d.get("random_feature_block_order", "true") == "true",
                       key_range=Range(0, max(1, space.n_cols)))
    hb = darlin_heap_bytes(cfg, world)
    fab = Fabric.from_process_group(hb) if world > 1 else Fabric.single(hb, dev)
    # the block kernels see column indices as keys; the column space is their identity list
    r = DarlinRank(fab, cfg, col.to(torch.int64), torch.from_numpy(y).to(dev), row_ptr=row_ptr, vals=vals,
                   global_keys=torch.arange(space.n_cols, dtype=torch.int64, device=dev))
    r.set_blocks(plan.blocks, plan.prior)
    if init_type != "ZERO":
        # the same vector on every rank: a constant, or draws of one seeded generator over the column space
        if init_type == "CONSTANT":
            w0 = np.full(space.n_cols, float(init_w.get("constant", 1)), np.float32)
        else:
            w0 = np.random.RandomState(20141010).normal(float(init_w.get("mean", 0)), float(init_w.get("std", 1)),
                                                        space.n_cols).astype(np.float32)
        r.set_initial_weights(torch.from_numpy(w0))

    def all_reduce(vals_, op):
        if dist is None:
            return vals_
        t = torch.tensor(vals_, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
        return t.tolist()

    out = conf.get("model_output", {}).get("file")
    out = (out if isinstance(out, str) else out[0]) if out else None

    def save(suffix=""):
        if not out:
            return
        cols_, w = r.my_model()
        keys = space.col_key[torch.from_numpy(cols_.astype(np.int64)).to(dev)].cpu().numpy().view(np.uint64)
        os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
        write_model(f"{out}{suffix}_S{rank}", keys, w)

    n_ex = int(all_reduce([float(len(y))], "sum")[0])
    if rank == 0 and verbose:
        print(f"  {n_ex} examples, {space.n_cols} features in {len(space.groups)} group(s), {len(plan.blocks)} blocks"
              + (f", tail filter dropped {space.dropped_nnz} local nonzeros" if tail else ""))
        print("  iter |  objective    relative   |w|_0   | violation  active set")
    hist = drive([r], all_reduce=all_reduce if dist is not None else None, verbose=verbose and rank == 0, num_examples=n_ex,
                 save_every=int(d.get("save_model_every_n_iter", 0)), save_fn=lambda it: save(f"_iter_{it}"))
    save()
    if dist is not None:
        dist.barrier()
        fab.close()
    return hist


def main(argv: Optional[List[str]] = None):
    ap = argparse.ArgumentParser(prefix_chars="-")
    ap.add_argument("-app_file", "--app_file", default="")
    ap.add_argument("-app_conf", "--app_conf", default="")
    ap.add_argument("-checkpoint_in", "--checkpoint_in", default="",
                    help="async SGD: resume from the binary shard checkpoint <prefix>_S<rank>.psbckpt")
    ap.add_argument("-checkpoint_out", "--checkpoint_out", default="",
                    help="async SGD: write weights and optimiser state to <prefix>_S<rank>.psbckpt at the end")
    ap.add_argument("-engine", "--engine", default="gpu", choices=["gpu", "null"],
                    help="null: run the node layer of async SGD (scheduler, workloads, leases, membership) without a device")
    ap.add_argument("-hash_kernel", "--hash_kernel", type=int, default=0, help=">0: feature ids are taken modulo this")
    ap.add_argument("-shuffle_fea_id", "--shuffle_fea_id", action="store_true", help="TERAFEA ids are mixed by a hash")
    ap.add_argument("-line_limit", "--line_limit", type=int, default=0, help=">0: lines read per text file")
    ap.add_argument("-num_threads", "--num_threads", type=int, default=0, help="threads that parse a text minibatch (default 2)")
    args, _ = ap.parse_known_args(argv)
    if args.hash_kernel or args.shuffle_fea_id or args.line_limit or args.num_threads:
        core.set_reader_flags(args.hash_kernel, args.shuffle_fea_id, args.line_limit, args.num_threads)
    text = (open(args.app_file).read() if args.app_file else "") + args.app_conf
    conf = core.parse_text_proto(text)
    conf["_checkpoint_in"], conf["_checkpoint_out"] = args.checkpoint_in, args.checkpoint_out
    if args.engine == "null":
        return run_async_sgd(conf, engine="null")
    from .. import _build
    _build.build_cuda()
    if "darlin" in conf:
        return run_darlin(conf)
    if "async_sgd" in conf:
        return run_async_sgd(conf)
    if "validation_data" in conf:
        return run_evaluation(conf)
    raise SystemExit("the configuration selects no application (async_sgd, darlin or validation_data)")


if __name__ == "__main__":
    main()
