"""Dense layers shared through the servers: every worker pushes its gradient of three layers, the servers add
them up (small layers live whole on one server, the large one is split evenly over both), and a worker pulls
the sums back with a pull that waits for its own push (the counterpart of the reference's
``src/test/kv_layer_ps.cc``).

    python examples/kv/kv_layer.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parameter_server_b200.system import LocalCluster, core  # noqa: E402

PARTITION_THRESHOLD = 100      # layers with more values than this are split over the servers
LAYERS = {0: 10, 1: 64, 2: 1000}   # layer id (the key channel of the requests) -> number of values


class Node(core.App):
    def __init__(self, po):
        super().__init__(po)
        self.layers = core.KVLayerSum(PARTITION_THRESHOLD, 9, po)     # an updater that adds what is pushed


def main():
    cluster = LocalCluster(2, 2, lambda conf, po: Node(po))
    try:
        workers = cluster.apps("W")
        pushed = {}
        for rank, w in enumerate(workers):
            for layer, n in LAYERS.items():
                gradient = np.full(n, rank + 1, dtype=np.float32)
                pushed[rank, layer] = w.layers.push(core.request(layer), gradient)
        for (rank, layer), ts in pushed.items():
            workers[rank].layers.wait(ts)
        sums = {}
        w0 = workers[0]
        for layer, n in LAYERS.items():
            out = np.zeros(n, np.float32)
            w0.layers.wait(w0.layers.pull(core.request(layer, -1, [pushed[0, layer]]), out))
            sums[layer] = out
            print(f"layer {layer}: {n} values, every one {out[0]:g}")      # 1 + 2 = 3
        parts = [len(s.layers.layer(2)) for s in cluster.apps("S")]
        print("the large layer is held as", parts)                         # [500, 500]
        return sums, parts
    finally:
        cluster.stop()


if __name__ == "__main__":
    main()
