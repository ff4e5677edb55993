"""Job control for CPU nodes, the counterpart of the reference's ``script/ps.sh``
(``start [-hostfile f] [-nw N] [-ns N] bin args`` / ``ls`` / ``add -worker N -server N`` /
``kill <id>`` / ``stop``, ``script/ps.sh:1-454``) and ``script/local.sh``.

Nodes are OS processes running ``bin`` (by default the in-tree ``bin/psb_linear``) with
``-my_node``, ``-scheduler``, ``-num_servers`` and ``-num_workers`` appended. Without a
host file every node runs on this machine (127.0.0.1); with one (one host per line) the
nodes are spread round-robin over the hosts and started through ``ssh host 'cmd'``, as
the reference does. The job's state (node ids, hosts, ports, pids with their start
times, the command) is kept in a JSON file inside a directory that only the user can
enter (``$XDG_RUNTIME_DIR/psb`` or ``~/.cache/psb``, mode 0700) so that later calls
(``ls``, ``add``, ``kill``, ``stop``) find the job. A state file that is not a regular
file owned by the caller is refused, and a process is only ever signalled when it is
still the one that was started (same pid *and* same start time), so a stale file or a
recycled pid cannot direct a signal at an unrelated process;
``add`` registers new nodes with the running scheduler and ``kill`` ends one node's
process, which is how elasticity and node failures are exercised.

    python -m parameter_server_b200.system.launch start -ns 2 -nw 2 -- bin/psb_linear -app_file x.conf
    python -m parameter_server_b200.system.launch ls
    python -m parameter_server_b200.system.launch add -worker 1
    python -m parameter_server_b200.system.launch kill W1
    python -m parameter_server_b200.system.launch stop
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import signal
import subprocess
import sys
import time
from typing import Dict, List, Optional

from .cluster import node_string


def _private_dir() -> str:
    """A directory only this user can enter: $XDG_RUNTIME_DIR/psb, else ~/.cache/psb (created 0700)."""
    base = os.environ.get("XDG_RUNTIME_DIR")
    if not base or not os.path.isdir(base) or os.stat(base).st_uid != os.getuid():
        base = os.path.join(os.path.expanduser("~"), ".cache")
    d = os.path.join(base, "psb")
    os.makedirs(d, mode=0o700, exist_ok=True)
    st = os.stat(d)
    if st.st_uid != os.getuid():
        raise PermissionError(f"{d} belongs to another user")
    if st.st_mode & 0o077:
        os.chmod(d, 0o700)
    return d


def default_state_path() -> str:
    return os.environ.get("PSB_STATE") or os.path.join(_private_dir(), "job.json")


def _start_time(pid: int) -> Optional[int]:
    """Start time of a process in clock ticks since boot (field 22 of /proc/<pid>/stat), None if gone."""
    try:
        with open(f"/proc/{pid}/stat") as f:
            return int(f.read().rsplit(")", 1)[1].split()[19])
    except (OSError, IndexError, ValueError):
        return None


def _free_port() -> int:
    import socket
    s = socket.socket()
    s.bind(("", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _alive(pid: int, started: Optional[int] = None) -> bool:
    """Is the process that was started as ``pid`` (at start time ``started``, if recorded) still running?"""
    try:
        os.kill(pid, 0)
    except OSError:
        return False
    # a finished child that nobody has waited for still answers signal 0
    try:
        with open(f"/proc/{pid}/stat") as f:
            if f.read().split(")")[-1].split()[0] == "Z":
                return False
    except OSError:
        return False
    return started is None or _start_time(pid) == started


def _node_alive(n: Dict) -> bool:
    return _alive(n["pid"], n.get("started"))


class Job:
    """One running job and its state file."""

    def __init__(self, path: Optional[str] = None):
        self.path = path or default_state_path()
        self.state: Dict = {}
        if os.path.lexists(self.path):
            # never act on a file somebody else could have planted
            st = os.lstat(self.path)
            import stat as _stat
            if not _stat.S_ISREG(st.st_mode) or st.st_uid != os.getuid():
                raise PermissionError(f"state file {self.path} is not a regular file owned by uid {os.getuid()}")
            with open(self.path) as f:
                self.state = json.load(f)

    # ------------------------------------------------------------------ helpers
    def _save(self):
        tmp = self.path + f".{os.getpid()}.tmp"
        fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o600)
        with os.fdopen(fd, "w") as f:
            json.dump(self.state, f, indent=1)
        os.replace(tmp, self.path)

    def _spawn(self, node_id: str, role: str, host: str, port: int) -> Dict:
        st = self.state
        spec = node_string(role, host, port, node_id)
        cmd = list(st["argv"]) + ["-my_node", spec, "-scheduler", st["scheduler"], "-num_servers", str(st["num_servers"]),
                                  "-num_workers", str(st["num_workers"])]
        log = os.path.join(st["log_dir"], f"{node_id}.log")
        out = open(log, "ab")
        if host in ("127.0.0.1", "localhost"):
            p = subprocess.Popen(cmd, stdout=out, stderr=subprocess.STDOUT, start_new_session=True)
        else:
            remote = "cd " + shlex.quote(st["cwd"]) + " && exec " + " ".join(shlex.quote(c) for c in cmd)
            # -tt: the remote process is tied to this ssh session and ends with it
            # host keys are checked as the user's ssh configuration says (no override here)
            p = subprocess.Popen(["ssh", "-tt", host, remote], stdout=out,
                                 stdin=subprocess.DEVNULL, stderr=subprocess.STDOUT, start_new_session=True)
        out.close()
        node = {"id": node_id, "role": role, "host": host, "port": port, "pid": p.pid, "log": log,
                "started": _start_time(p.pid)}
        st["nodes"].append(node)
        return node

    def _hosts(self) -> List[str]:
        return self.state.get("hosts") or ["127.0.0.1"]

    def _next_index(self, prefix: str) -> int:
        used = [int(n["id"][1:]) for n in self.state["nodes"] if n["id"].startswith(prefix) and n["id"][1:].isdigit()]
        return max(used) + 1 if used else 0

    # ------------------------------------------------------------------ commands
    def start(self, argv: List[str], num_servers: int, num_workers: int, hostfile: Optional[str] = None,
              log_dir: Optional[str] = None):
        if self.state.get("nodes") and any(_node_alive(n) for n in self.state["nodes"]):
            raise RuntimeError(f"a job is already running (state file {self.path}); stop it first")
        hosts = None
        if hostfile:
            with open(hostfile) as f:
                hosts = [h.strip() for h in f if h.strip() and not h.startswith("#")]
        log_dir = log_dir or os.path.join(_private_dir(), f"logs-{int(time.time())}")
        os.makedirs(log_dir, mode=0o700, exist_ok=True)
        sched_host = (hosts or ["127.0.0.1"])[0]
        sched_port = _free_port()
        self.state = {"argv": argv, "num_servers": num_servers, "num_workers": num_workers, "hosts": hosts,
                      "scheduler": node_string("SCHEDULER", sched_host, sched_port, "H"), "nodes": [],
                      "log_dir": log_dir, "cwd": os.getcwd()}
        self._spawn("H", "SCHEDULER", sched_host, sched_port)
        hs = self._hosts()
        k = 1
        for i in range(num_servers):
            self._spawn(f"S{i}", "SERVER", hs[k % len(hs)], _free_port()); k += 1
        for i in range(num_workers):
            self._spawn(f"W{i}", "WORKER", hs[k % len(hs)], _free_port()); k += 1
        self._save()
        return self.state["nodes"]

    def ls(self) -> List[Dict]:
        return [dict(n, alive=_node_alive(n)) for n in self.state.get("nodes", [])]

    def add(self, workers: int = 0, servers: int = 0) -> List[Dict]:
        """Start more nodes; they register with the running scheduler (REGISTER_NODE)."""
        if not self.state:
            raise RuntimeError("no job")
        hs = self._hosts()
        new = []
        for _ in range(servers):
            i = self._next_index("S")
            new.append(self._spawn(f"S{i}", "SERVER", hs[i % len(hs)], _free_port()))
        for _ in range(workers):
            i = self._next_index("W")
            new.append(self._spawn(f"W{i}", "WORKER", hs[i % len(hs)], _free_port()))
        self._save()
        return new

    def kill(self, node_id: str, sig: int = signal.SIGKILL) -> bool:
        """End one node's process (a node failure, as seen by the others)."""
        for n in self.state.get("nodes", []):
            if n["id"] == node_id:
                # the recorded pid is the node itself (local) or its ssh session (remote node); it leads
                # its own session (start_new_session), so the group id is the pid. Signal it only if it
                # is still the process that was started.
                if not _node_alive(n):
                    return False
                try:
                    if os.getpgid(n["pid"]) != n["pid"]:
                        return False
                    os.killpg(n["pid"], sig)
                except OSError:
                    return False
                return True
        raise KeyError(node_id)

    def wait(self, timeout: Optional[float] = None) -> bool:
        """Wait until no node is alive; True if the job ended in time."""
        t0 = time.time()
        while any(_node_alive(n) for n in self.state.get("nodes", [])):
            for n in self.state["nodes"]:      # reap our own finished children
                try:
                    os.waitpid(n["pid"], os.WNOHANG)
                except OSError:
                    pass
            if timeout is not None and time.time() - t0 > timeout:
                return False
            time.sleep(0.05)
        return True

    def stop(self):
        for n in self.state.get("nodes", []):
            if _node_alive(n):
                try:
                    self.kill(n["id"], signal.SIGTERM)
                except (OSError, KeyError):
                    pass
        self.wait(5)
        for n in self.state.get("nodes", []):
            if _node_alive(n):
                try:
                    self.kill(n["id"], signal.SIGKILL)
                except (OSError, KeyError):
                    pass
        self.wait(5)
        if os.path.exists(self.path):
            os.remove(self.path)
        self.state = {}


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m parameter_server_b200.system.launch")
    ap.add_argument("--state", default=None, help="state file (default: $PSB_STATE, else job.json in a private per-user directory)")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("start")
    s.add_argument("-ns", type=int, default=1); s.add_argument("-nw", type=int, default=1)
    s.add_argument("-hostfile", default=None); s.add_argument("-log_dir", default=None)
    s.add_argument("argv", nargs=argparse.REMAINDER, help="-- bin args...")
    sub.add_parser("ls")
    s = sub.add_parser("add"); s.add_argument("-worker", type=int, default=0); s.add_argument("-server", type=int, default=0)
    s = sub.add_parser("kill"); s.add_argument("id")
    sub.add_parser("stop")
    s = sub.add_parser("wait"); s.add_argument("-timeout", type=float, default=None)
    s = sub.add_parser("root-node", help="print the -scheduler string for this machine (script/get_root_node.sh)")
    s.add_argument("interface", help="network interface whose address the scheduler binds, e.g. eth0; '' = first one")
    s.add_argument("port", type=int)
    a = ap.parse_args(argv)
    if a.cmd == "root-node":
        from . import core
        from .cluster import node_string
        print(node_string("SCHEDULER", core.local_ip(a.interface), a.port, "H"))
        return 0
    job = Job(a.state)
    if a.cmd == "start":
        cmd = [c for c in a.argv if c != "--"]
        if not cmd:
            ap.error("start needs the node binary and its arguments after --")
        for n in job.start(cmd, a.ns, a.nw, a.hostfile, a.log_dir):
            print(f"{n['id']:4s} {n['role']:9s} {n['host']}:{n['port']} pid {n['pid']} log {n['log']}")
    elif a.cmd == "ls":
        for n in job.ls():
            print(f"{n['id']:4s} {n['role']:9s} {n['host']}:{n['port']} pid {n['pid']} {'alive' if n['alive'] else 'gone'}")
    elif a.cmd == "add":
        for n in job.add(a.worker, a.server):
            print(f"{n['id']:4s} {n['role']:9s} {n['host']}:{n['port']} pid {n['pid']}")
    elif a.cmd == "kill":
        job.kill(a.id)
    elif a.cmd == "wait":
        return 0 if job.wait(a.timeout) else 1
    elif a.cmd == "stop":
        job.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
