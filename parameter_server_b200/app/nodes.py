"""GPU ranks as parameter-server nodes.

One process per GPU hosts a server node ``S<r>`` (the rank's key-range shard) and
a worker node ``W<r>``; rank 0 also hosts the scheduler ``H``. The nodes are
ordinary nodes of the C++ host runtime (``csrc/core``): they register with the
scheduler's manager, exchange ``Task`` headers through their customers'
executors, and learn about lost nodes from the manager. Bulk data never takes
this path: keys, weights and gradients move between the GPUs inside the fused
kernels; only headers travel on the host.

The message flow of asynchronous SGD is the reference's
(``learner/sgd.cc:8-49``, ``app/linear_method/async_sgd.h:202-257``):

* a worker asks for work (``REQUEST_WORKLOAD``); the scheduler hands out one
  file of the training set at a time from its ``WorkloadPool``
  (``UPDATE_MODEL`` with a ``Workload``), the worker answers when the file is
  done and gets the next one; a lost worker's files go back into the pool;
* workers and servers report progress to the scheduler's monitor customer
  (``system/monitor.h:17-97``), which prints the progress table;
* at the end the scheduler asks the servers to write the model (``SAVE_MODEL``).

One addition: the device shards aggregate round ``t`` of all workers before
the optimiser runs, so every rank runs every round (with an empty minibatch
when it has no data). The scheduler therefore grants rounds in leases
(``ROUND_LIMIT``, see ``LockstepSGDScheduler`` in ``csrc/core/learner.h``) and
the limit in force when the last file is finished is where every rank stops.
No collective and no host synchronisation happens per minibatch.
"""
from __future__ import annotations

import os
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import numpy as np

from ..system import core
from ..system.cluster import node_string


class Engine:
    """What the node layer needs from the thing that trains. ``GpuEngine`` in
    ``app/linear.py`` drives the device data plane; :class:`NullEngine` only
    counts, for tests of the control flow on machines without a GPU."""

    def submit(self, batch) -> int:
        """Run one lock-step round; ``batch`` is ``(labels, csr dict)`` from the
        stream reader or ``None`` for an empty round. Returns the number of rows."""
        raise NotImplementedError

    def finish(self):
        """Block until every submitted round has completed."""

    def progress(self) -> dict:
        """Counters since the last call: ``loss_sum, n_correct, n_examples, auc,
        d_nnz, weight_sum, delta_sum``."""
        return {}

    def set_alive(self, rank: int, alive: bool):
        """Membership change learned from the manager."""

    def save_model(self, path: str):
        """Write this rank's shard as ``key<TAB>weight`` lines."""


class NullEngine(Engine):
    def __init__(self, step_seconds: float = 0.0):
        self.rounds, self.rows, self.new_rows = 0, 0, 0
        self.alive_calls: List[tuple] = []
        self.saved: List[str] = []
        self.step_seconds = step_seconds

    def submit(self, batch) -> int:
        n = 0 if batch is None else len(batch[0])
        self.rounds += 1
        self.rows += n
        self.new_rows += n
        if self.step_seconds:
            time.sleep(self.step_seconds)
        return n

    def progress(self) -> dict:
        n, self.new_rows = self.new_rows, 0
        return {"loss_sum": 0.6931 * n, "n_correct": 0.5 * n, "n_examples": n, "auc": 0.5, "d_nnz": 0,
                "weight_sum": 0.0, "delta_sum": 0.0}

    def set_alive(self, rank: int, alive: bool):
        self.alive_calls.append((rank, alive))

    def save_model(self, path: str):
        self.saved.append(path)
        with open(path, "w") as f:
            f.write("")


def make_reader(files: List[str], data_format: str, text: str):
    """The minibatch source of a workload: mapped binary matrices for ``format: BIN`` (no parsing), the C++
    stream reader for text and record files. Both give ``read_matrices(n) -> (labels, [csr dict]) | None``."""
    if data_format == "BIN":
        from ..utils.binfmt import BinReader
        return BinReader(files)
    return core.StreamReader(files, data_format, text, True)


class TailFeatureFilter:
    """Drops rare features from the minibatches before they reach the device: the loader-side count-min
    filter of the reference's ``MinibatchReader`` (``learner/sgd.h:88-91,123-134``). Every minibatch adds the
    counts of its unique keys to the sketch (saturating 8-bit cells); a nonzero stays when its key's estimated
    count so far is greater than ``freq``. ``countmin_n`` cells, ``countmin_k`` hash functions
    (``async_sgd { tail_feature_freq countmin_n countmin_k }``)."""

    def __init__(self, freq: int, countmin_n: float = 1e8, countmin_k: int = 2):
        self.freq = int(freq)
        self.filter = core.FreqencyFilter()
        self.filter.resize(int(min(max(countmin_n, 1024), 1 << 30)), int(countmin_k))
        self.dropped = 0

    def apply(self, batch):
        """``batch``: ``(labels, [csr dict per slot])`` from the stream reader; returns the same with the
        filtered nonzeros taken out (rows keep their places, some may become empty)."""
        y, mats = batch
        out = []
        for m in mats:
            keys = np.ascontiguousarray(m["index"], dtype=np.uint64)
            uniq, cnt = np.unique(keys, return_counts=True)
            self.filter.insert_keys(uniq, np.minimum(cnt, 255).astype(np.uint8))
            kept = self.filter.query_keys(uniq, self.freq)
            mask = np.isin(keys, kept, assume_unique=False)
            if mask.all():
                out.append(m)
                continue
            self.dropped += int(len(keys) - mask.sum())
            off = np.asarray(m["offset"], dtype=np.int64)
            new_off = np.concatenate([[0], np.cumsum(mask, dtype=np.int64)])[off].astype(np.uint64)
            f = dict(m)
            f["offset"], f["index"] = new_off, keys[mask]
            if not m["binary"] and len(m["value"]):
                f["value"] = np.asarray(m["value"])[mask]
            out.append(f)
        return y, out


@dataclass
class _Workload:
    ids: List[int]
    files: List[str]
    request: object            # the UPDATE_MODEL message, answered when the file is done


class RankState:
    """Shared between the node threads (executor callbacks) and the rank's main loop."""

    def __init__(self):
        self.cv = threading.Condition()
        self.limit = 0
        self.final = False
        self.final_request = None
        self.workloads: "queue.Queue[_Workload]" = queue.Queue()
        self.commands: "queue.Queue[tuple]" = queue.Queue()
        self.shutdown = threading.Event()      # set by the main loop: this rank's nodes may leave the job

    def set_limit(self, limit: int, final: bool, request=None):
        with self.cv:
            self.limit = max(self.limit, limit)
            if final:
                self.final = True
                self.final_request = request
            self.cv.notify_all()

    def wait_round(self, t: int, timeout: float = 600.0):
        """Block until round ``t`` is granted or the job is closed. Returns True if ``t`` may run."""
        deadline = time.time() + timeout
        with self.cv:
            while t >= self.limit and not self.final:
                left = deadline - time.time()
                if left <= 0:
                    raise TimeoutError(f"no round lease beyond {self.limit} from the scheduler")
                self.cv.wait(min(left, 1.0))
            return t < self.limit


class LockstepWorkerApp(core.App):
    """The worker node's application: asks for workloads, queues them for the
    rank's main loop, keeps the round lease."""

    def __init__(self, po, state: RankState):
        core.App.__init__(self, po)
        self.po, self.state = po, state
        self.reporter = core.SGDReporter(po)

    def run(self):
        t = core.Task()
        t.sgd_cmd = core.SGD_REQUEST_WORKLOAD
        self.submit(t, self.po.scheduler_node().id)

    def process_request(self, m):
        task = m.task
        if not task.has_sgd:
            return
        if task.sgd_cmd == core.SGD_UPDATE_MODEL:
            m.finished = False                      # answered by finish_workload() when the file is done
            self.state.workloads.put(_Workload(list(task.sgd_load_ids), list(task.sgd_load_files), m))
        elif task.sgd_cmd == core.SGD_ROUND_LIMIT:
            if task.sgd_final_round:
                m.finished = False                  # answered by ack_final() after the last round
                self.state.set_limit(task.sgd_round_limit, True, m)
            else:
                self.state.set_limit(task.sgd_round_limit, False)

    def finish_workload(self, w: _Workload):
        done = core.Task()
        done.sgd_cmd = core.SGD_UPDATE_MODEL
        done.sgd_load_ids = w.ids
        done.sgd_load_finished = True
        self.finish_received_request(w.request.task.time, w.request.sender)
        self.reply(w.request, done)

    def ack_final(self):
        req = self.state.final_request
        if req is not None:
            self.finish_received_request(req.task.time, req.sender)
            self.reply(req)


class ShardServerApp(core.App):
    """The server node's application. The shard itself lives on the GPU; on
    ``SAVE_MODEL`` the rank's main loop (which owns the device) writes it."""

    def __init__(self, po, state: RankState):
        core.App.__init__(self, po)
        self.po, self.state = po, state
        self.reporter = core.SGDReporter(po)

    def process_request(self, m):
        if m.task.has_sgd and m.task.sgd_cmd == core.SGD_SAVE_MODEL:
            done = threading.Event()
            self.state.commands.put(("save", self.po.my_node().id, done))
            done.wait(600)


@dataclass
class RankNodes:
    """The postoffices of this rank and the threads that run them."""
    state: RankState
    threads: List[threading.Thread] = field(default_factory=list)
    offices: dict = field(default_factory=dict)
    errors: List[BaseException] = field(default_factory=list)
    worker: Optional[LockstepWorkerApp] = None
    server: Optional[ShardServerApp] = None
    scheduler: Optional[object] = None

    def alive(self) -> bool:
        return any(t.is_alive() for t in self.threads)


def scheduler_spec(host: str, port: int) -> str:
    return node_string("SCHEDULER", host, port, "H")


def start_rank_nodes(rank: int, world: int, sched_spec: str, *, files: List[str], data_format: str = "TEXT",
                     text: str = "LIBSVM", passes: int = 1, lease: int = 64, roles: str = "HSW",
                     on_node_lost: Optional[Callable[[str], None]] = None, host: str = "127.0.0.1",
                     inproc: bool = False) -> RankNodes:
    """Start this rank's nodes, each on its own thread: register and run the app (``Postoffice.run``),
    then, once the rank's main loop is through (the scheduler: once its ``Run`` has returned), tell
    the scheduler that the node is ready to exit and stay until it says so (``Postoffice.stop``).
    ``roles`` selects among scheduler (H, rank 0 only), server (S) and worker (W). ``inproc`` puts
    the nodes of a single-process job on the in-process van."""
    state = RankState()
    nodes = RankNodes(state)

    def factory(conf, po):
        role = po.my_node().role
        if role == core.Node.Role.SCHEDULER:
            nodes.scheduler = core.LockstepSGDScheduler(files, data_format, text, passes, True, lease, po)
            return nodes.scheduler
        if role == core.Node.Role.WORKER:
            nodes.worker = LockstepWorkerApp(po, state)
            return nodes.worker
        nodes.server = ShardServerApp(po, state)
        return nodes.server

    core.set_app_factory(factory)
    specs = []
    h = "inproc" if inproc else host
    if rank == 0 and "H" in roles:
        specs.append(("H", sched_spec))
    if "S" in roles:
        specs.append((f"S{rank}", node_string("SERVER", h, (sched_port(sched_spec) + 1 + rank) if inproc else core.free_port(), f"S{rank}")))
    if "W" in roles:
        specs.append((f"W{rank}", node_string("WORKER", h, (sched_port(sched_spec) + 1000 + rank) if inproc else core.free_port(), f"W{rank}")))
    n_servers = int(os.environ.get("PSB_NUM_SERVERS", world))
    n_workers = int(os.environ.get("PSB_NUM_WORKERS", world))

    def run_node(nid, po, opt):
        try:
            po.run(opt)
            if nid != "H":
                state.shutdown.wait()
            po.stop()
        except BaseException as e:  # noqa: BLE001  (reported by the main loop)
            nodes.errors.append(e)

    for nid, spec in specs:
        po = core.Postoffice()
        opt = core.Options()
        opt.num_servers, opt.num_workers = n_servers, n_workers
        opt.my_node, opt.scheduler = spec, sched_spec
        opt.app_conf = "lockstep"
        opt.exit_on_scheduler_loss = False
        if on_node_lost is not None and nid != "H":
            po.add_node_failure_handler(on_node_lost)
        nodes.offices[nid] = po
        th = threading.Thread(target=run_node, args=(nid, po, opt), name=f"ps-{nid}", daemon=True)
        nodes.threads.append(th)
        th.start()
    return nodes


def sched_port(spec: str) -> int:
    return int(spec.split("port:")[1].split(",")[0])


def node_rank(node_id: str) -> Optional[int]:
    """Rank of the process that hosts node ``S<r>`` / ``W<r>``."""
    if len(node_id) > 1 and node_id[0] in "SW" and node_id[1:].isdigit():
        return int(node_id[1:])
    return None


def run_lockstep_worker_loop(nodes: RankNodes, engine: Engine, *, minibatch: int, data_format: str = "TEXT",
                             text: str = "LIBSVM", report_interval: float = 1.0, model_file: Optional[str] = None,
                             idle_wait: float = 0.0005, start_timeout: float = 120.0, save_timeout: float = 600.0,
                             after_round: Optional[Callable[[int], None]] = None, announce: str = "",
                             tail_filter: Optional["TailFeatureFilter"] = None) -> dict:
    """The rank's main loop: rounds ``0, 1, ...`` while the scheduler's lease allows, a minibatch of
    the current workload per round (an empty round when there is none), progress reports, and at
    the end the commands of the rank's server node (model dump). Returns counters."""
    state = nodes.state
    t0 = time.time()
    while nodes.worker is None or (nodes.server is None and any(k.startswith("S") for k in nodes.offices)):
        if nodes.errors:
            raise nodes.errors[0]
        if time.time() - t0 > start_timeout:
            raise TimeoutError("this rank's nodes did not start")
        time.sleep(0.001)
    wapp, sapp = nodes.worker, nodes.server
    t = 0
    cur: Optional[_Workload] = None
    reader = None
    examples = 0
    files_done = 0
    nnz_w = 0
    last_report = time.time()
    last_round_report = 0

    def report(final=False):
        nonlocal nnz_w
        p = engine.progress()
        n = p.get("n_examples", 0)
        nnz_w = max(0, nnz_w + int(p.get("d_nnz", 0)))
        if n > 0 or final:
            wapp.reporter.report(objective=[p.get("loss_sum", 0.0)], accuracy=[p.get("n_correct", 0.0) / max(1.0, n)],
                                 auc=[p.get("auc", 0.5)], num_examples=int(n), round=t)
        if sapp is not None:
            sapp.reporter.report(nnz=nnz_w, weight_sum=p.get("weight_sum", 0.0), delta_sum=p.get("delta_sum", 0.0))

    while True:
        if nodes.errors:
            raise nodes.errors[0]
        if not state.wait_round(t):
            break
        batch = None
        while True:
            if cur is None:
                try:
                    cur = state.workloads.get(timeout=idle_wait) if idle_wait else state.workloads.get_nowait()
                except queue.Empty:
                    break
                reader = make_reader(cur.files, data_format, text)
                if announce and files_done == 0:
                    print(f"{announce} first workload {cur.files[0]}", flush=True)
            got = reader.read_matrices(minibatch)
            if got is None:
                wapp.finish_workload(cur)           # the scheduler marks the file done and sends the next one
                cur, reader = None, None
                files_done += 1
                continue
            if len(got[0]) and got[1]:
                batch = got if tail_filter is None else tail_filter.apply(got)
                break
        examples += engine.submit(batch)
        t += 1
        if after_round is not None:
            after_round(t)
        now = time.time()
        if t - last_round_report >= 8:
            # the scheduler keeps the lease ahead of the largest round it has heard of
            wapp.reporter.report(round=t)
            last_round_report = t
        if now - last_report >= report_interval:
            last_report = now
            report()
    engine.finish()
    report(final=True)
    wapp.ack_final()
    # the server node's command (the scheduler asks every server to write its part of the model once
    # all workers have answered the final lease); after it this rank's nodes may leave the job
    deadline = time.time() + save_timeout
    while sapp is not None and time.time() < deadline:
        if nodes.errors:
            raise nodes.errors[0]
        try:
            cmd = state.commands.get(timeout=0.05)
        except queue.Empty:
            continue
        if cmd[0] == "save":
            if model_file:
                os.makedirs(os.path.dirname(model_file) or ".", exist_ok=True)
                engine.save_model(f"{model_file}_{cmd[1]}")
            cmd[2].set()
            break
    state.shutdown.set()
    for th in nodes.threads:
        th.join(timeout=30)
    if nodes.errors:
        raise nodes.errors[0]
    return {"rounds": t, "examples": examples, "files": files_done}
