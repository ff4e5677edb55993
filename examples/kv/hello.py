"""The smallest parameter-server program: one scheduler, two servers and two workers in this process;
a worker submits a task to the server group, waits for it and is called back (the counterpart of the
reference's ``src/test/hello_ps.cc``).

    python examples/kv/hello.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parameter_server_b200.system import LocalCluster, core  # noqa: E402


class Hello(core.App):
    """Servers print what they are asked; every node runs one of these."""

    def __init__(self, po):
        super().__init__(po)
        self.me = po.my_node().id

    def process_request(self, msg):
        print(f"{self.me}: request {msg.task.time} from {msg.sender}: {bytes(msg.task.msg).decode()}")


def main():
    cluster = LocalCluster(2, 2, lambda conf, po: Hello(po))
    try:
        worker = cluster.app("W0")
        task = core.Task()
        task.msg = b"hello world"
        msg = core.Message(task)
        msg.recver = core.kServerGroup                      # every server gets a copy
        msg.callback = lambda: print("W0: every server has answered")
        ts = worker.submit_message(msg)
        worker.wait(ts)                                     # returns after the callback has run
        ts2 = worker.submit(task, "S1")                     # one recipient
        worker.wait(ts2)
        print("W0: last response came from", worker.last_response().sender)
        return ts, ts2
    finally:
        cluster.stop()


if __name__ == "__main__":
    main()
