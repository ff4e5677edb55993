"""The socket transport under two stress programs (tests/cpp), run as OS processes over TCP on 127.0.0.1."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def programs(tmp_path_factory):
    from parameter_server_b200 import _build
    lib, _ = _build.build_static()
    out = tmp_path_factory.mktemp("transport")
    cxx = os.environ.get("PSB_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    exes = {}
    for name in ("order_check", "bidir_big"):
        exes[name] = str(out / name)
        subprocess.run([cxx, "-O1", "-std=c++17", "-pthread", "-I", os.path.join(ROOT, "parameter_server_b200", "csrc", "core"),
                        os.path.join(ROOT, "tests", "cpp", name + ".cc"), str(lib), "-lz", "-o", exes[name]],
                       check=True, timeout=600)
    return exes


def test_requests_of_a_node_arrive_in_timestamp_order(programs):
    """Two threads submit 3000 small requests each without waiting; whether a message is written by the submitting
    thread or by the send thread, the server sees increasing timestamps and every request is acknowledged."""
    from parameter_server_b200.system.cluster import launch_local_processes
    for _ in range(3):
        out = launch_local_processes(1, 1, [programs["order_check"]], timeout=120)
        assert all(p.returncode == 0 for p in out.values()), {k: (p.returncode, p.stdout[-300:]) for k, p in out.items()}
        assert "ORDER OK 6000" in out["S0"].stdout and "ACKED 6000" in out["W0"].stdout


def test_large_messages_in_both_directions_complete(programs):
    """Pushes and pulls of a million keys issued back to back by two workers against two servers: outgoing data
    and replies fill the socket buffers at the same time. A thread that holds its executor's lock must never
    wait in a write (two nodes doing that to each other stop reading for good); this run hangs if one does."""
    from parameter_server_b200.system.cluster import launch_local_processes
    for _ in range(3):
        out = launch_local_processes(2, 2, [programs["bidir_big"]], timeout=60)
        assert all(p.returncode == 0 for p in out.values()), {k: (p.returncode, p.stdout[-300:]) for k, p in out.items()}
        assert all("DONE 6" in out[w].stdout for w in ("W0", "W1"))
