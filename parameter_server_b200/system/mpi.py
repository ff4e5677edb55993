"""Start a job with ``mpirun``: the counterpart of the reference's ``script/mpi_root.sh`` and
``script/mpi_node.sh``.

    python -m parameter_server_b200.system.mpi root mpi.conf          # on the first machine
    (mpirun then runs, once per rank:)
    python -m parameter_server_b200.system.mpi node <scheduler> mpi.conf

``mpi.conf`` is a file of ``name=value`` lines (shell syntax, as the reference sources it):
``num_workers``, ``num_servers``, ``bin``, ``arg``, ``network_interface``, ``network_port`` and
optionally ``hostfile``. ``root`` works out this machine's address on ``network_interface``, builds
the scheduler's node string and execs ``mpirun -np 1+servers+workers``; ``node`` reads its rank from
the MPI launcher's environment (MPICH ``PMI_RANK`` / Open MPI ``OMPI_COMM_WORLD_RANK``) and execs the
node binary: rank 0 is the scheduler, ranks 1..num_servers are servers, the rest workers.
"""
from __future__ import annotations

import os
import shlex
import sys
from typing import Dict, List, Optional

from .cluster import node_string


def read_conf(path: str) -> Dict[str, str]:
    """``name=value`` lines; quotes as in a shell, ``#`` comments."""
    out: Dict[str, str] = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#") or "=" not in line:
                continue
            name, _, value = line.partition("=")
            parts = shlex.split(value, comments=True)
            out[name.strip()] = " ".join(parts)
    return out


def mpi_rank_and_size(env=os.environ):
    for r, s in (("PMI_RANK", "PMI_SIZE"), ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE")):
        if r in env and s in env:
            return int(env[r]), int(env[s])
    raise RuntimeError("neither PMI_RANK/PMI_SIZE nor OMPI_COMM_WORLD_RANK/OMPI_COMM_WORLD_SIZE is set: "
                       "start this through mpirun")


def root_command(conf_path: str, conf: Dict[str, str], local_ip: str) -> List[str]:
    """The ``mpirun`` command line of ``mpi_root.sh``."""
    n = int(conf["num_workers"]) + int(conf["num_servers"]) + 1
    sched = node_string("SCHEDULER", local_ip, int(conf.get("network_port", "8000")), "H")
    cmd = ["mpirun"]
    if conf.get("hostfile"):
        cmd += ["-hostfile", conf["hostfile"]]
    cmd += ["-np", str(n), sys.executable, "-m", "parameter_server_b200.system.mpi", "node", sched, conf_path]
    return cmd


def node_command(scheduler: str, conf: Dict[str, str], rank: int, size: int, local_ip: str, port: int) -> List[str]:
    """The node binary's command line for MPI rank ``rank`` (``mpi_node.sh``)."""
    ns, nw = int(conf["num_servers"]), int(conf["num_workers"])
    if size < ns + nw + 1:
        raise RuntimeError(f"too small rank size {size}: {ns} servers + {nw} workers + the scheduler need {ns + nw + 1}")
    if rank == 0:
        me = scheduler
    elif rank <= ns:
        me = node_string("SERVER", local_ip, port, f"S{rank - 1}")
    else:
        me = node_string("WORKER", local_ip, port, f"W{rank - ns - 1}")
    cmd = shlex.split(conf["bin"]) + ["-num_servers", str(ns), "-num_workers", str(nw), "-scheduler", scheduler,
                                      "-my_node", me]
    if conf.get("network_interface"):
        cmd += ["-interface", conf["network_interface"]]
    return cmd + shlex.split(conf.get("arg", ""))


def main(argv: Optional[List[str]] = None) -> int:
    from . import core
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) >= 2 and argv[0] == "root":
        conf = read_conf(argv[1])
        cmd = root_command(argv[1], conf, core.local_ip(conf.get("network_interface", "")))
    elif len(argv) >= 3 and argv[0] == "node":
        conf = read_conf(argv[2])
        rank, size = mpi_rank_and_size()
        cmd = node_command(argv[1], conf, rank, size, core.local_ip(conf.get("network_interface", "")), core.free_port())
    else:
        print(__doc__)
        return 2
    if "--dry-run" in argv:
        print(" ".join(shlex.quote(c) for c in cmd))
        return 0
    os.execvp(cmd[0], cmd)
    return 1


if __name__ == "__main__":
    sys.exit(main())
