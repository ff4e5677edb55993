"""Device KV containers as customers of the host runtime (parameter/kv_nodes.py): the message flow on
in-process nodes with a recording backend, and (on a GPU) real containers on two emulated ranks."""
import threading
import time

import numpy as np
import pytest

from parameter_server_b200.system import LocalCluster, core


class _Rec:
    """Stands in for the device: records what the customers ask of it."""

    def __init__(self, name, events):
        self.name, self.events, self.rounds = name, events, 0

    def push(self, keys, values):
        self.rounds += 1
        self.events.append(("push", self.name, self.rounds - 1))
        return self.rounds - 1

    def apply(self, rnd):
        self.events.append(("apply", self.name, rnd))

    def pull(self, keys):
        self.events.append(("pull", self.name))
        return list(keys)

    def set_alive(self, rank, alive):
        self.events.append(("alive", self.name, rank, alive))


def _cluster(events):
    from parameter_server_b200.parameter.kv_nodes import KVServerCustomer, KVWorkerCustomer

    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            me = po.my_node()
            if me.role == core.Node.Role.SERVER:
                self.kv = KVServerCustomer(po, 9, _Rec(me.id, events), ["W0", "W1"])
            elif me.role == core.Node.Role.WORKER:
                self.kv = KVWorkerCustomer(po, 9, _Rec(me.id, events))

    return LocalCluster(2, 2, lambda conf, po: A(po))


def test_round_is_merged_when_every_worker_has_pushed_and_dependent_pull_waits_for_it():
    events = []
    cl = _cluster(events)
    try:
        w0, w1 = (a.kv for a in cl.apps("W"))
        got = {}

        def first_worker():
            tp = w0.push([1, 2], [1.0, 2.0])
            tq = w0.pull([1, 2], wait=[tp])
            w0.wait(tq)
            got["w0"] = (tp, tq, w0.result(tq), time.time())

        th = threading.Thread(target=first_worker)
        th.start()
        time.sleep(0.5)
        # W1 has not pushed: no server has merged round 0, and W0's dependent pull is still held back
        assert not [e for e in events if e[0] == "apply"] and "w0" not in got
        t_push = time.time()
        tp1 = w1.push([3], [3.0])
        w1.wait(tp1)                                  # answered once both servers merged the round
        th.join(10)
        assert got["w0"][2] == [1, 2] and got["w0"][1] == got["w0"][0] + 1 and got["w0"][3] >= t_push
        applies = [e for e in events if e[0] == "apply"]
        assert sorted(applies) == [("apply", "S0", 0), ("apply", "S1", 0)]
        # on every server: both push headers were processed before W0's pull header
        for s in cl.apps("S"):
            kinds = [(k, snd) for k, snd, _ in s.kv.log]
            assert kinds.index(("pull", "W0")) > kinds.index(("push", "W1"))
        # the pull kernel ran after the merges had been launched
        assert events.index(("pull", "W0")) > max(events.index(a) for a in applies)
    finally:
        cl.stop()


def test_callback_fires_once_all_servers_answered_and_lost_worker_is_not_waited_for():
    events = []
    cl = _cluster(events)
    try:
        w0, w1 = (a.kv for a in cl.apps("W"))
        fired = []
        tp = w0.push([5], [1.0], callback=lambda: fired.append("pushed"))
        time.sleep(0.3)
        assert fired == []                            # W1's push of the round is missing
        cl.nodes["H"].node_disconnected("W1")         # the scheduler learns that W1 is gone and tells every node
        w0.wait(tp)
        assert fired == ["pushed"]
        assert sorted(e for e in events if e[0] == "apply") == [("apply", "S0", 0), ("apply", "S1", 0)]
        assert ("alive", "S0", 1, False) in events
    finally:
        cl.stop()


@pytest.mark.gpu
def test_device_containers_behind_node_customers(cuda_lib):
    """Two emulated ranks on one GPU, every rank a server node and a worker node of an in-process job:
    pushes go through the kernels, their headers through the executors; the owners merge a round when
    both headers are there; a pull that waits for the push returns the sums."""
    import torch
    from parameter_server_b200.parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig, heap_layout
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.parameter.kv import DeviceKVVector
    from parameter_server_b200.parameter.kv_nodes import DeviceKVBackend, KVServerCustomer, KVWorkerCustomer
    pc = PlaneConfig(table_capacity=1 << 12, inbox_cap=256, ring=4, pull_cap=0)
    fabs = Fabric.emulated(2, heap_layout(pc, 2).total())
    kvs = [DeviceKVVector(DataPlane(f, pc, OptimizerConfig(algo="sum")), 256) for f in fabs]
    for kv in kvs:                                     # emulated ranks share the GPU: one stream keeps their kernels in order
        kv.stream = torch.cuda.current_stream()
    backends = [DeviceKVBackend(kv) for kv in kvs]

    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            me = po.my_node()
            r = int(me.id[1:]) if me.id[1:].isdigit() else 0
            if me.role == core.Node.Role.SERVER:
                self.kv = KVServerCustomer(po, 9, backends[r], ["W0", "W1"])
            elif me.role == core.Node.Role.WORKER:
                self.kv = KVWorkerCustomer(po, 9, backends[r])

    cl = LocalCluster(2, 2, lambda conf, po: A(po))
    try:
        half = 1 << 63
        keys = np.array([3, 9, half + 4], dtype=np.uint64)
        ws = sorted(cl.apps("W"), key=lambda a: a.my_node().id)
        stamps = [w.kv.push(keys, np.array([1.0, 2.0, 3.0], np.float32) * (i + 1)) for i, w in enumerate(ws)]
        tq = ws[0].kv.pull(keys, wait=[stamps[0]])
        ws[0].kv.wait(tq)
        out = ws[0].kv.result(tq)
        torch.cuda.synchronize()
        assert out.cpu().tolist() == [3.0, 6.0, 9.0]
        for kv in kvs:
            kv.plane.check_status()
    finally:
        cl.stop()
