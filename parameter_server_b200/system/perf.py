"""Throughput probes of the host runtime, the counterparts of the reference's three perf programs
over its own transport:

* ``network``   raw message throughput worker -> servers: requests that carry ``--data-size`` KB of
                payload, ``--n`` of them, acknowledged by the servers (``test/network_perf_ps.cc:23-47``);
* ``kv_map``    ``KVMap`` push of random keys with gaussian values, then a pull that depends on the
                push (``test/kv_map_perf_ps.cc:27-60``);
* ``kv_layer``  ``KVLayer`` push + dependent pull of the AlexNet layer sizes
                (``test/kv_layer_perf_ps.cc:34-70``).

All nodes (scheduler, ``-ns`` servers, ``-nw`` workers) run in this process over the in-process van,
like ``script/local.sh`` with ``-local``; the numbers are MB/s of payload per worker. The device-side
probes are in ``parameter_server_b200.ops.microbench`` (``fabric``, ``kv``, ``layer``).

    python -m parameter_server_b200.system.perf network --data-size 1024 --n 100
"""
from __future__ import annotations

import argparse
import json
import threading
import time

import numpy as np

ALEXNET_LAYERS = [11 * 11 * 3 * 32, 5 * 5 * 16 * 16, 3 * 3 * 284, 3 * 3 * 256, 13 * 13 * 256 * 4096 // 64, 4096 * 4096 // 16,
                  4096 * 1000]   # the two largest are scaled down: a host probe, not a memory test


def _cluster(ns, nw, factory):
    from . import LocalCluster
    return LocalCluster(ns, nw, factory)


def network(args):
    from . import core

    class Sink(core.App):
        def __init__(self, po):
            super().__init__(po)

        def process_request(self, msg):      # the reply (an empty acknowledgement) is sent by the executor
            pass

    cl = _cluster(args.ns, args.nw, lambda conf, po: Sink(po))
    try:
        payload = bytes(args.data_size * 1024)
        out = []

        def work(w):
            t = core.Task()
            t.msg = payload
            t0 = time.perf_counter()
            last = -1
            for _ in range(args.n):
                last = w.submit(t, core.kServerGroup)
            w.wait(last)
            out.append(time.perf_counter() - t0)
        th = [threading.Thread(target=work, args=(w,)) for w in cl.apps("W")]
        [t.start() for t in th]
        [t.join() for t in th]
        sec = max(out)
        mb = args.n * args.ns * args.data_size / 1024.0
        return {"probe": "network", "servers": args.ns, "workers": args.nw, "KB_per_message": args.data_size, "messages": args.n,
                "MB_per_s_per_worker": mb / sec, "seconds": sec}
    finally:
        cl.stop()


def kv_map(args):
    from . import core

    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            if po.my_node().role == core.Node.Role.SERVER:
                self.kv = core.KVMapSum(1, 9, po)
            else:
                self.kv = core.KVVector(False, 1, 9, po)

    cl = _cluster(args.ns, args.nw, lambda conf, po: A(po))
    try:
        out = []

        def work(i, w):
            rng = np.random.default_rng(i)
            keys = np.unique(rng.integers(0, 1 << 63, args.keys, dtype=np.uint64) * np.uint64(2))
            vals = rng.normal(size=len(keys)).astype(np.float32)
            w.kv.set_channel(0, keys, np.zeros(len(keys), np.float32))
            t0 = time.perf_counter()
            for _ in range(args.n):
                ts = w.kv.push(core.request(0), keys, [vals])
                w.kv.wait(w.kv.pull(core.request(0, -1, [ts]), keys))      # the pull depends on the push
            out.append((time.perf_counter() - t0, len(keys)))
        th = [threading.Thread(target=work, args=(i, w)) for i, w in enumerate(cl.apps("W"))]
        [t.start() for t in th]
        [t.join() for t in th]
        sec = max(o[0] for o in out)
        nk = out[0][1]
        mb = args.n * nk * (8 + 4 + 8 + 4) / 1e6          # keys + values out, keys out + values back
        return {"probe": "kv_map", "servers": args.ns, "workers": args.nw, "keys": nk, "rounds": args.n,
                "MB_per_s_per_worker": mb / sec, "keys_per_s_per_worker": 2 * args.n * nk / sec, "seconds": sec}
    finally:
        cl.stop()


def kv_layer(args):
    from . import core

    class A(core.App):
        def __init__(self, po):
            super().__init__(po)
            self.kv = core.KVLayerSum(args.partition_thr, 9, po)

    cl = _cluster(args.ns, args.nw, lambda conf, po: A(po))
    try:
        out = []

        def work(w):
            bufs = [np.random.default_rng(l).normal(size=n).astype(np.float32) for l, n in enumerate(ALEXNET_LAYERS)]
            outs = [np.zeros(n, np.float32) for n in ALEXNET_LAYERS]
            t0 = time.perf_counter()
            for _ in range(args.n):
                pulls = []
                for l, b in enumerate(bufs):
                    ts = w.kv.push(core.request(l), b)
                    pulls.append(w.kv.pull(core.request(l, -1, [ts]), outs[l]))
                for ts in pulls:
                    w.kv.wait(ts)
            out.append(time.perf_counter() - t0)
        th = [threading.Thread(target=work, args=(w,)) for w in cl.apps("W")]
        [t.start() for t in th]
        [t.join() for t in th]
        sec = max(out)
        mb = args.n * 2 * 4 * sum(ALEXNET_LAYERS) / 1e6
        return {"probe": "kv_layer", "servers": args.ns, "workers": args.nw, "layer_elements": ALEXNET_LAYERS, "rounds": args.n,
                "MB_per_s_per_worker": mb / sec, "seconds": sec}
    finally:
        cl.stop()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("network", "kv_map", "kv_layer"):
        s = sub.add_parser(name)
        s.add_argument("-ns", type=int, default=2)
        s.add_argument("-nw", type=int, default=2)
        s.add_argument("--n", type=int, default=20)
        if name == "network":
            s.add_argument("--data-size", type=int, default=1024, help="payload per message in KB")
        if name == "kv_map":
            s.add_argument("--keys", type=int, default=100000)
        if name == "kv_layer":
            s.add_argument("--partition-thr", type=int, default=1000)
    args = ap.parse_args(argv)
    res = {"network": network, "kv_map": kv_map, "kv_layer": kv_layer}[args.cmd](args)
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
