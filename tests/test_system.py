"""Host runtime semantics, re-expressing the reference's multi-process test
programs (src/test/hello_ps.cc, aggregation_ps.cc, kv_vector_ps.cc,
kv_vector_buffer_ps.cc, kv_map_ps.cc, kv_layer_ps.cc) as assertions, with all
nodes inside one process (in-process van)."""
import threading
import time

import numpy as np
import pytest

from parameter_server_b200.system import LocalCluster, core


class Recorder(core.App):
    """Records every request it processes."""

    def __init__(self, po):
        super().__init__(po)
        self.po = po
        self.seen = []
        self.lock = threading.Lock()

    def process_request(self, msg):
        with self.lock:
            self.seen.append((msg.sender, msg.task.time, bytes(msg.task.msg)))


def test_range_even_divide_matches_long_double():
    from parameter_server_b200.utils.range import Range
    r = core.KeyRange.all()
    for n in (1, 2, 3, 7, 8):
        for i in range(n):
            a, b = r.even_divide(n, i), Range.all().even_divide(n, i)
            assert (a.begin, a.end) == (b.begin, b.end)
    assert core.KeyRange(10, 20).set_intersection(core.KeyRange(15, 30)) == core.KeyRange(15, 20)


def test_task_wire_roundtrip():
    t = core.Task()
    t.request, t.customer_id, t.time, t.wait_time = True, 7, 42, [40, 41]
    t.key_range = core.KeyRange(5, 99)
    t.key_channel, t.msg, t.more = 3, b"hello\x00world", True
    t.filter = [core.FilterConfig(core.FilterConfig.Type.FIXING_FLOAT, num_bytes=2)]
    u = core.Task.parse(t.serialize())
    assert (u.request, u.customer_id, u.time, u.wait_time, u.key_channel, u.more) == (True, 7, 42, [40, 41], 3, True)
    assert u.key_range == core.KeyRange(5, 99) and bytes(u.msg) == b"hello\x00world"
    assert u.filter[0].type == core.FilterConfig.Type.FIXING_FLOAT and u.filter[0].num_bytes == 2


def test_slice_message_by_key_range():
    m = core.Message()
    keys = np.array([1, 5, 9, 20, 21, 40], dtype=np.uint64)
    m.set_key(keys)
    m.add_value(np.arange(12, dtype=np.float32))  # k = 2
    t = m.task
    t.key_range = core.KeyRange(0, 30)
    m.task = t
    parts = core.slice_message(m, [core.KeyRange(0, 10), core.KeyRange(10, 20), core.KeyRange(20, 30), core.KeyRange(30, 50)])
    assert [p.valid for p in parts] == [True, True, True, False]
    assert parts[0].key().tolist() == [1, 5, 9] and parts[0].value(0).tolist() == [0, 1, 2, 3, 4, 5]
    assert parts[1].key().tolist() == []               # owned range without keys: valid and empty
    assert parts[2].key().tolist() == [20, 21] and parts[2].value(0).tolist() == [6, 7, 8, 9]


def test_hello_submit_wait_callback():
    cl = LocalCluster(2, 2, lambda conf, po: Recorder(po), conf="hello")
    try:
        w0, w1 = cl.apps("W")
        done = []
        t = core.Task()
        t.msg = b"hi"
        m = core.Message(t)
        m.recver = core.kServerGroup
        m.callback = lambda: done.append(1)
        ts = w0.submit_message(m)
        w0.wait(ts)
        assert done == [1]
        ts2 = w0.submit(t, core.kServerGroup)
        assert ts2 == ts + 1
        w0.wait(ts2)
        for s in cl.apps("S"):
            assert [(x[0], x[2]) for x in s.seen] == [("W0", b"hi"), ("W0", b"hi")]
        # a single recipient, and the response is visible
        ts3 = w1.submit(t, "S1")
        w1.wait(ts3)
        assert w1.last_response().sender == "S1"
        assert [x[0] for x in cl.app("S1").seen].count("W1") == 1
        # the two servers split the key space (ranges follow registration order, not node ids)
        lo, hi = sorted((a.my_node().key for a in cl.apps("S")), key=lambda k: k.begin)
        assert lo.end == hi.begin
    finally:
        cl.stop()


def test_wait_time_dependencies_order_execution():
    """A request that waits on timestamp t runs only after t is finished, even if it arrives first."""
    class Slow(Recorder):
        def process_request(self, msg):
            if bytes(msg.task.msg) == b"slow":
                time.sleep(0.15)
            super().process_request(msg)

    cl = LocalCluster(1, 1, lambda conf, po: Slow(po))
    try:
        w = cl.app("W0")
        a = core.Task(); a.msg = b"slow"; a.time = 5
        b = core.Task(); b.msg = b"after"; b.time = 3; b.wait_time = [5]
        c = core.Task(); c.msg = b"free"; c.time = 4
        # b is submitted first but depends on a
        tb = w.submit(b, "S0"); tc = w.submit(c, "S0"); ta = w.submit(a, "S0")
        for t in (ta, tb, tc):
            w.wait(t)
        order = [x[2] for x in cl.app("S0").seen]
        assert order.index(b"slow") < order.index(b"after")
        assert order[0] == b"free"
    finally:
        cl.stop()


def test_aggregation_wait_received_request_on_worker_group():
    """Server-side barrier: WaitReceivedRequest(t, kWorkerGroup) returns once every worker's t arrived."""
    cl = LocalCluster(1, 3, lambda conf, po: Recorder(po))
    try:
        s = cl.app("S0")
        got = []

        def server():
            for i in range(4):
                s.wait_received_request(i, core.kWorkerGroup)
                got.append((i, s.num_done_received_request(i, core.kWorkerGroup)))
        th = threading.Thread(target=server)
        th.start()
        for i in range(4):
            for w in cl.apps("W"):
                t = core.Task(); t.time = i
                w.submit(t, core.kServerGroup)
        th.join(timeout=20)
        assert got == [(0, 3), (1, 3), (2, 3), (3, 3)]
    finally:
        cl.stop()


def test_virtual_timestamp_releases_dependent_request():
    """Push at t, server finishes virtual t+1, pull at t+2 waiting on t+1 (the aggregation idiom)."""
    class Holder(Recorder):
        pass

    cl = LocalCluster(1, 2, lambda conf, po: Holder(po))
    try:
        s = cl.app("S0")
        ws = cl.apps("W")
        for w in ws:
            a = core.Task(); a.time = 0; a.msg = b"push"
            w.submit(a, core.kServerGroup)
            b = core.Task(); b.time = 2; b.wait_time = [1]; b.msg = b"pull"
            w.submit(b, core.kServerGroup)
        s.wait_received_request(0, core.kWorkerGroup)
        time.sleep(0.1)
        assert [x[2] for x in s.seen] == [b"push", b"push"]      # pulls are held back
        s.finish_received_request(1, core.kWorkerGroup)
        for w in ws:
            w.wait(2)
        assert sorted(x[2] for x in s.seen) == [b"pull", b"pull", b"push", b"push"]
    finally:
        cl.stop()


def test_deferred_finish_blocks_wait_until_app_finishes():
    class Deferring(Recorder):
        def process_request(self, msg):
            super().process_request(msg)
            if self.my_node().role == core.Node.Role.SERVER:
                msg.finished = False
                self.pending = (msg.task.time, msg.sender)
                self.pending_msg = msg

    cl = LocalCluster(1, 1, lambda conf, po: Deferring(po))
    try:
        w, s = cl.app("W0"), cl.app("S0")
        ts = w.submit(core.Task(), "S0")
        flag = []
        th = threading.Thread(target=lambda: (w.wait(ts), flag.append(1)))
        th.start()
        time.sleep(0.2)
        assert flag == [] and s.num_done_received_request(ts, "W0") == 0
        req = s.last_request()
        s.finish_received_request(ts, "W0")
        s.reply(req)
        th.join(timeout=10)
        assert flag == [1]
    finally:
        cl.stop()


def test_task_packing_more_flag_delivers_all_in_order():
    cl = LocalCluster(1, 1, lambda conf, po: Recorder(po))
    try:
        w, s = cl.app("W0"), cl.app("S0")
        sent0 = cl.nodes["W0"].sent_bytes()
        last = None
        for i in range(20):
            t = core.Task(); t.msg = b"%d" % i; t.more = i < 19
            last = w.submit(t, "S0")
        w.wait(last)
        for i in range(last - 19, last):
            w.wait(i)
        assert [x[2] for x in s.seen] == [b"%d" % i for i in range(20)]
    finally:
        cl.stop()


def _servers_by_range(cl):
    """Servers ordered by the key range they own (ranges are handed out in registration
    order, which need not be the order of the node ids)."""
    return sorted(cl.apps("S"), key=lambda a: a.my_node().key.begin)


def test_kv_vector_push_pull_two_channels():
    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            self.kv = core.KVVector(False, 1, 9, po)

    cl = LocalCluster(2, 2, lambda conf, po: A(po))
    try:
        half = 1 << 63
        all_keys = np.array([1, 3, 5, half + 2, half + 4, half + 8], dtype=np.uint64)
        for s in cl.apps("S"):
            for chl in (0, 1):
                s.kv.set_channel(chl, all_keys, (np.arange(6) + 10 * chl).astype(np.float32))
        w0, w1 = cl.apps("W")
        k0 = np.array([1, 5, half + 4], dtype=np.uint64)
        k1 = np.array([3, half + 2, half + 8], dtype=np.uint64)
        w0.kv.set_channel(0, k0, np.zeros(3, np.float32))
        w1.kv.set_channel(1, k1, np.zeros(3, np.float32))
        w0.kv.wait(w0.kv.pull(core.request(0), k0))
        w1.kv.wait(w1.kv.pull(core.request(1), k1))
        assert w0.kv.values(0).tolist() == [0, 2, 4]
        assert w1.kv.values(1).tolist() == [11, 13, 15]
        # push adds into the servers' values
        w0.kv.wait(w0.kv.push(core.request(0), k0, [np.ones(3, np.float32)]))
        s0, s1 = _servers_by_range(cl)
        assert s0.kv.values(0).tolist()[:3] == [1, 1, 3] and s1.kv.values(0).tolist()[4] == 5
    finally:
        cl.stop()


def test_kv_vector_buffered_aggregation_and_dependent_pull():
    """Two value arrays (k=2) pushed by every worker at ts, summed in the server's
    buffer(ts); the server publishes a result and finishes virtual ts+1; workers
    pull at ts+2 waiting on ts+1."""
    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            self.kv = core.KVVector(True, 2, 9, po)

    cl = LocalCluster(2, 3, lambda conf, po: A(po))
    try:
        half = 1 << 63
        keys = np.array([2, 4, half + 1, half + 3], dtype=np.uint64)
        for w in cl.apps("W"):
            w.kv.set_channel(4, keys, np.zeros(8, np.float32))
        for j, s in enumerate(_servers_by_range(cl)):     # every server holds the keys of its own range
            s.kv.set_channel(4, keys[2 * j:2 * j + 2], np.zeros(4, np.float32))
        ts = 0
        for i, w in enumerate(cl.apps("W")):
            g = np.full(8, 1.0 + i, np.float32)
            u = np.full(8, 10.0 * (1 + i), np.float32)
            w.kv.push(core.request(4, ts), keys, [g, u])
            w.kv.pull(core.request(4, ts + 2, [ts + 1]), keys)
        for j, s in enumerate(_servers_by_range(cl)):
            s.kv.wait_received_request(ts, core.kWorkerGroup)
            buf = s.kv.buffer(ts)
            assert buf["idx_range"] == (0, 2) and buf["channel"] == 4
            assert buf["values"][0].tolist() == [6.0] * 4 and buf["values"][1].tolist() == [60.0] * 4
            s.kv.set_channel(4, keys[2 * j:2 * j + 2], buf["values"][0] + buf["values"][1])
            s.kv.finish_received_request(ts + 1, core.kWorkerGroup)
        for w in cl.apps("W"):
            w.kv.wait(ts + 2)
            b = w.kv.buffer(ts + 2)
            assert b["idx_range"] == (0, 4) and b["values"][0].tolist() == [66.0] * 8
    finally:
        cl.stop()


def test_kv_map_custom_entry_push_then_pull():
    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            self.role = po.my_node().role
            if self.role == core.Node.Role.SERVER:
                self.kv = core.KVMapSum(1, 9, po)
            else:
                self.kv = core.KVVector(False, 1, 9, po)

    cl = LocalCluster(2, 2, lambda conf, po: A(po))
    try:
        half = 1 << 63
        keys = np.array([7, 9, half + 5], dtype=np.uint64)
        ws = cl.apps("W")
        for i, w in enumerate(ws):
            w.kv.set_channel(0, keys, np.zeros(3, np.float32))
            w.kv.wait(w.kv.push(core.request(0), keys, [np.array([1, 2, 3], np.float32) * (i + 1)]))
        w = ws[0]
        w.kv.wait(w.kv.pull(core.request(0), keys))
        assert w.kv.values(0).tolist() == [3, 6, 9]
        assert [s.kv.size() for s in _servers_by_range(cl)] == [2, 1]
    finally:
        cl.stop()


def test_kv_layer_small_and_partitioned_layers():
    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            self.kv = core.KVLayerSum(100, 9, po)

    cl = LocalCluster(2, 2, lambda conf, po: A(po))
    try:
        ws = cl.apps("W")
        sizes = {0: 10, 1: 64, 2: 1000}
        for lid, n in sizes.items():
            for i, w in enumerate(ws):
                w.kv.wait(w.kv.push(core.request(lid), np.arange(n, dtype=np.float32) * (i + 1)))
        for lid, n in sizes.items():
            out = np.zeros(n, np.float32)
            w = ws[lid % 2]
            w.kv.wait(w.kv.pull(core.request(lid), out))
            assert np.allclose(out, np.arange(n) * 3.0), lid
        # the large layer is split over both servers, small ones live on one
        s0, s1 = cl.apps("S")
        assert len(s0.kv.layer(2)) == 500 and len(s1.kv.layer(2)) == 500
        assert sorted([len(s0.kv.layer(0)), len(s1.kv.layer(0))]) == [0, 10]
    finally:
        cl.stop()


def test_dead_node_completes_waits_and_drops_its_messages():
    cl = LocalCluster(2, 2, lambda conf, po: Recorder(po))
    try:
        fails = []
        cl.nodes["H"].add_node_failure_handler(lambda nid: fails.append(nid))
        s0 = cl.app("S0")
        th_done = []
        th = threading.Thread(target=lambda: (s0.wait_received_request(0, core.kWorkerGroup), th_done.append(1)))
        th.start()
        t = core.Task(); t.time = 0
        cl.app("W0").submit(t, core.kServerGroup)
        time.sleep(0.2)
        assert th_done == []                      # W1 has not sent timestamp 0
        cl.nodes["H"].node_disconnected("W1")     # host-side failure injection at the scheduler
        th.join(timeout=10)
        assert th_done == [1] and fails == ["W1"]
        assert cl.nodes["S0"].num_workers() == 1 and s0.num_alive(core.kWorkerGroup) == 1
        # a request to the worker group now only targets W0
        ts = s0.submit(core.Task(), core.kWorkerGroup)
        s0.wait(ts)
        assert [x[0] for x in cl.app("W0").seen] == ["S0"]
    finally:
        cl.stop()
