"""Push and pull with the shared key-value vector: two workers add values under their keys, the servers
(each owns half of the key space) sum them, and a worker pulls the sums back with a pull that waits for
its own push (the counterpart of the reference's ``src/test/kv_vector_ps.cc`` and ``kv_map_ps.cc``).

    python examples/kv/kv_vector.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parameter_server_b200.system import LocalCluster, core  # noqa: E402


class Node(core.App):
    def __init__(self, po):
        super().__init__(po)
        if po.my_node().role == core.Node.Role.SERVER:
            self.kv = core.KVMapSum(1, 9, po)            # entries that add what is pushed
        else:
            self.kv = core.KVVector(False, 1, 9, po)     # one value per key, customer id 9 on every node


def main():
    cluster = LocalCluster(2, 2, lambda conf, po: Node(po))
    try:
        half = 1 << 63
        keys = np.array([7, 9, half + 5], dtype=np.uint64)          # two keys on the first server, one on the second
        workers = cluster.apps("W")
        stamps = []
        for i, w in enumerate(workers):
            w.kv.set_channel(0, keys, np.zeros(len(keys), np.float32))
            stamps.append(w.kv.push(core.request(0), keys, [np.array([1, 2, 3], np.float32) * (i + 1)]))
        for w, ts in zip(workers, stamps):
            w.kv.wait(ts)
        w0 = workers[0]
        w0.kv.wait(w0.kv.pull(core.request(0, -1, [stamps[0]]), keys))   # the pull waits for this worker's push
        print("pulled", w0.kv.values(0).tolist())                       # [3.0, 6.0, 9.0]
        return w0.kv.values(0).tolist()
    finally:
        cluster.stop()


if __name__ == "__main__":
    main()
