"""Start a whole parameter-server system inside one process.

The reference tests multi-node behaviour by launching real processes on
localhost (``script/local.sh:10-44``). :class:`LocalCluster` does the same with
one :class:`Postoffice` per node and the in-process van, each node on its own
thread, which makes multi-node semantics (timestamps, dependencies, groups, node
death) unit-testable; :func:`launch_local_processes` is the multi-process,
TCP-socket equivalent of ``local.sh``.
"""
from __future__ import annotations

import os
import subprocess
import sys
import threading
from typing import Callable, Dict, List, Optional

_counter = [0]
_lock = threading.Lock()


def node_string(role: str, host: str, port: int, node_id: str) -> str:
    return f"role:{role},hostname:'{host}',port:{port},id:'{node_id}'"


class LocalCluster:
    """Scheduler ``H`` + servers ``S0..`` + workers ``W0..`` in this process.

    ``factory(conf, po)`` must return the :class:`App` of the node that owns the
    postoffice ``po`` (look at ``po.my_node().role``).
    """

    def __init__(self, num_servers: int, num_workers: int, factory: Optional[Callable], conf: str = "",
                 key_start: int = 0, key_end: Optional[int] = None, run: bool = False, num_threads: int = 2):
        """``factory=None`` selects the C++ linear-method applications (from ``conf``).
        With ``run=True`` every node also runs its app's ``Run()`` (the scheduler's
        returns when the job is done); call :meth:`join` to wait for it."""
        from . import core
        self.core = core
        self._run = run
        with _lock:
            _counter[0] += 1
            base = _counter[0] * 1000
        if factory is None:
            core.use_linear_method_factory()
        else:
            core.set_app_factory(factory)
        sched = node_string("SCHEDULER", "inproc", base, "H")
        specs = [("H", sched)]
        specs += [(f"S{i}", node_string("SERVER", "inproc", base + 1 + i, f"S{i}")) for i in range(num_servers)]
        specs += [(f"W{i}", node_string("WORKER", "inproc", base + 500 + i, f"W{i}")) for i in range(num_workers)]
        self.nodes: Dict[str, object] = {}
        self._threads: List[threading.Thread] = []
        self._errors: List[BaseException] = []
        for nid, spec in specs:
            po = core.Postoffice()
            opt = core.Options()
            opt.num_servers, opt.num_workers = num_servers, num_workers
            opt.my_node, opt.scheduler, opt.app_conf = spec, sched, conf
            opt.exit_on_scheduler_loss = False
            opt.num_threads = num_threads
            if key_end is not None:
                opt.key_start, opt.key_end = key_start, key_end
            self.nodes[nid] = po
            t = threading.Thread(target=self._start, args=(po, opt), name=f"ps-{nid}", daemon=True)
            self._threads.append(t)
        if run:
            for t in self._threads:
                t.start()
            return
        # the scheduler first: everybody connects to it
        self._threads[0].start()
        self._threads[0].join()
        for t in self._threads[1:]:
            t.start()
        for t in self._threads[1:]:
            t.join()
        if self._errors:
            raise self._errors[0]
        for po in self.nodes.values():
            po.wait_servers_ready()
            po.wait_workers_ready()

    def _start(self, po, opt):
        try:
            if self._run:
                po.run(opt)
            else:
                po.start(opt)
        except BaseException as e:  # noqa: BLE001
            self._errors.append(e)

    def join(self, timeout: Optional[float] = None):
        """Wait until every node's ``Run()`` has returned (``run=True``)."""
        for t in self._threads:
            t.join(timeout)
        if self._errors:
            raise self._errors[0]

    def app(self, node_id: str):
        return self.nodes[node_id].app()

    def apps(self, prefix: str):
        return [self.app(n) for n in sorted(self.nodes, key=lambda s: (len(s), s)) if n.startswith(prefix)]

    def stop(self):
        ts = [threading.Thread(target=po.stop, daemon=True) for po in self.nodes.values()]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=30)


def launch_local_processes(num_servers: int, num_workers: int, argv: List[str], *, base_port: Optional[int] = None,
                           env: Optional[dict] = None, local_ipc: bool = False, timeout: float = 300.0,
                           capture: bool = True):
    """Run ``argv`` once per node as OS processes on 127.0.0.1, like the
    reference's ``script/local.sh <ns> <nw> <bin> [args]``. Every process gets
    ``-my_node``, ``-scheduler``, ``-num_servers`` and ``-num_workers``
    appended. Returns ``{node_id: CompletedProcess}``."""
    from . import core
    base = base_port or core.free_port()
    sched = node_string("SCHEDULER", "127.0.0.1", base, "H")
    specs = [("H", sched)]
    specs += [(f"S{i}", node_string("SERVER", "127.0.0.1", core.free_port(), f"S{i}")) for i in range(num_servers)]
    specs += [(f"W{i}", node_string("WORKER", "127.0.0.1", core.free_port(), f"W{i}")) for i in range(num_workers)]
    procs = {}
    for nid, spec in specs:
        cmd = list(argv) + ["-my_node", spec, "-scheduler", sched, "-num_servers", str(num_servers),
                            "-num_workers", str(num_workers)] + (["-local"] if local_ipc else [])
        procs[nid] = subprocess.Popen(cmd, env={**os.environ, **(env or {})},
                                      stdout=subprocess.PIPE if capture else None,
                                      stderr=subprocess.STDOUT if capture else None, text=True)
    # Every node's pipe is drained by its own thread: a node that prints more than a pipe holds
    # must not block while another node is being waited for. `timeout` bounds the whole job.
    out = {}

    def drain(nid, p):
        try:
            so, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            so, _ = p.communicate()
        out[nid] = subprocess.CompletedProcess(p.args, p.returncode, so, None)

    ts = [threading.Thread(target=drain, args=(nid, p), daemon=True) for nid, p in procs.items()]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return {nid: out[nid] for nid in procs}
