"""Device KV containers as customers of the host runtime.

``parameter/kv.py`` gives a container the reference's calling conventions with
CUDA events; here the same container is a pair of :class:`Customer` objects on a
rank's worker node and server node, and a Push or Pull is a request of the
executor: it gets the executor's timestamp, its ``wait`` list travels as the
task's ``wait_time`` and is enforced by the receiving executor, the callback
fires when every server has answered, and ``wait(ts)`` is the executor's wait
(``system/customer.h:170-199``, ``system/executor.cc:108-148,199-210``,
``parameter/kv_vector.h:245-262``). Only the header travels on the host; keys and
values move between the GPUs inside the kernels, as before.

What the server node adds is the reference's aggregation point
(``WaitReceivedRequest(t, kWorkerGroup)``, ``test/aggregation_ps.cc:7-30``): it
counts the push headers of every worker and merges round k (``backend.apply``)
when the k-th push of every live worker has arrived, so the owner's kernel is
launched when its inputs are on their way and never has to wait for a worker
that has not pushed yet. A pull that names a push in its ``wait`` list is held
back by the server's executor until that push has been processed there, i.e.
until the merge it belongs to has been launched; the worker then runs the pull
kernel (``backend.pull``) after every server has acknowledged.

The backend is what moves data: :class:`DeviceKVBackend` wraps a
:class:`~parameter_server_b200.parameter.kv.DeviceKVMap`; tests of the message
flow on machines without a GPU pass a recording stand-in.
"""
from __future__ import annotations

import threading
from typing import Callable, Dict, List, Optional, Sequence

from ..system import core


class DeviceKVBackend:
    """The device half behind a worker / server customer pair of one rank."""

    def __init__(self, kv):
        self.kv = kv

    def push(self, keys, values) -> int:
        return self.kv.push_only(keys, values)

    def apply(self, rnd: int):
        self.kv.apply_round(rnd)

    def pull(self, keys):
        ts = self.kv.pull(keys)
        self.kv.wait(ts)
        return self.kv.result(ts)

    def set_alive(self, rank: int, alive: bool):
        self.kv.plane.set_alive(rank, alive)


class KVServerCustomer(core.Customer):
    """Server node side: merges a push round once every live worker's header of that round is here."""

    def __init__(self, po, customer_id: int, backend, workers: Sequence[str]):
        core.Customer.__init__(self, customer_id, po)
        self.backend = backend
        self._lock = threading.Lock()
        self._pushed: Dict[str, int] = {w: 0 for w in workers}
        self._held: Dict[int, list] = {}              # round -> push requests not yet finished
        self.applied_rounds = 0
        self.log: List[tuple] = []                    # (kind, sender, time) in processing order
        # the manager tells every node when a node has left (system/manager.cc:250-270): a lost worker's
        # rounds are not waited for any more, and the data plane skips it as a source
        po.add_node_failure_handler(self._node_lost)

    def _node_lost(self, node_id: str):
        if node_id in self._pushed:
            self.worker_lost(node_id, rank=int(node_id[1:]) if node_id[1:].isdigit() else None)

    def process_request(self, m):
        kind = bytes(m.task.msg)[:4]
        done = []
        with self._lock:
            self.log.append((kind.decode(), m.sender, m.task.time))
            if kind == b"push":
                # the request stays unfinished until its round has been merged: a pull that waits for it is
                # then held back by the executor until the merge is launched (the deferred finish of the
                # reference's aggregation idiom, parameter/kv_vector.h:182-207)
                m.finished = False
                rnd = self._pushed.get(m.sender, 0)
                self._pushed[m.sender] = rnd + 1
                self._held.setdefault(rnd, []).append(m)
                done = self._merge_ready()
        # a pull header needs nothing here: its wait_time has kept it back until the pushes it names were
        # finished, and the empty reply that the executor sends is the acknowledgement the worker waits for
        self._release(done)

    def _merge_ready(self):
        """Merge every round that all live workers have pushed; returns the requests to finish (lock held)."""
        done = []
        ready = min(self._pushed.values()) if self._pushed else self.applied_rounds
        while self.applied_rounds < ready:
            self.backend.apply(self.applied_rounds)
            done += self._held.pop(self.applied_rounds, [])
            self.applied_rounds += 1
        return done

    def _release(self, requests):
        for req in requests:
            self.finish_received_request(req.task.time, req.sender)
            self.reply(req)

    def worker_lost(self, worker_id: str, rank: Optional[int] = None):
        """A worker has left the job: its rounds are no longer waited for."""
        with self._lock:
            self._pushed.pop(worker_id, None)
            if rank is not None:
                self.backend.set_alive(rank, False)
            done = self._merge_ready()
        self._release(done)


class KVWorkerCustomer(core.Customer):
    """Worker node side: ``push`` / ``pull`` / ``wait`` with the executor's timestamps."""

    def __init__(self, po, customer_id: int, backend):
        core.Customer.__init__(self, customer_id, po)
        self.backend = backend
        self._results: Dict[int, object] = {}
        self._pull_keys: Dict[int, object] = {}

    def _header(self, kind: bytes, wait: Sequence[int], callback: Optional[Callable]):
        t = core.Task()
        t.msg = kind
        t.wait_time = [int(w) for w in wait]
        m = core.Message(t)
        m.recver = core.kServerGroup
        if callback is not None:
            m.callback = callback
        return self.submit_message(m)

    def push(self, keys, values, wait: Sequence[int] = (), callback: Optional[Callable] = None) -> int:
        """Send this worker's values of the round to the owners (device) and the push header to every
        server (host). Returns the executor's timestamp."""
        self.backend.push(keys, values)
        return self._header(b"push", wait, callback)

    def pull(self, keys, wait: Sequence[int] = (), callback: Optional[Callable] = None) -> int:
        """Ask for the values of ``keys``; ``wait`` names earlier timestamps of this worker (usually the
        push before) that every server must have processed first. The values are there after :meth:`wait`."""
        ts = self._header(b"pull", wait, callback)
        self._pull_keys[ts] = keys
        return ts

    def wait(self, ts: int):
        """Block until every server has answered request ``ts``; a pull then runs its kernel."""
        core.Customer.wait(self, ts)
        keys = self._pull_keys.pop(ts, None)
        if keys is not None:
            self._results[ts] = self.backend.pull(keys)

    def result(self, ts: int):
        return self._results.pop(ts)
