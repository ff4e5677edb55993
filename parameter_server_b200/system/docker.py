"""Run a job as docker containers on this machine, one container per node: the counterpart of the
reference's ``docker/local.sh`` (and ``docker/build.sh``, ``docker/rm_local.sh``).

    python -m parameter_server_b200.system.docker build  [-image NAME]
    python -m parameter_server_b200.system.docker local  NUM_SERVERS NUM_WORKERS APP_CONF DATA_DIR MODEL_DIR [args...]
    python -m parameter_server_b200.system.docker rm     NUM_SERVERS NUM_WORKERS
    python -m parameter_server_b200.system.docker upload LOCAL_FILE s3://bucket/key

``local`` mounts the configuration at ``/app.conf``, the data at ``/data`` and the model directory at
``/model`` in every container and starts the scheduler on the docker bridge's address, port 8000, the
servers and workers on the ports after it, as the reference does. ``--dry-run`` prints the ``docker``
commands instead of running them. The image is built from ``docker/Dockerfile`` at the repository
root (CPU nodes: the C++ host runtime and ``bin/psb_linear``). The reference's EC2 / docker-machine
swarm scripts (``cloud.sh``, ``fire_amazonec2.sh``, ``shut.sh``) drive a tool that is no longer distributed
and are not rebuilt; ``upload`` is ``upload_s3.sh`` (one ``curl --upload-file`` to a public-read object).
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
from typing import List, Optional

from .cluster import node_string

IMAGE = "psb200/parameter-server"
BIN_IN_IMAGE = "/opt/psb/bin/psb_linear"


def bridge_ip() -> str:
    """Address of the docker0 bridge (what containers use to reach published ports of the host)."""
    try:
        out = subprocess.run(["ip", "-4", "-o", "addr", "show", "docker0"], capture_output=True, text=True, timeout=10).stdout
        return out.split("inet ")[1].split("/")[0].strip()
    except (OSError, IndexError, subprocess.SubprocessError):
        return "172.17.0.1"


def local_commands(num_servers: int, num_workers: int, app: str, data: str, model: str, extra: List[str],
                   ip: str, image: str = IMAGE, port: int = 8000) -> List[List[str]]:
    """One ``docker run`` command per node: scheduler n0, servers n1.., workers after them."""
    mounts = ["-v", f"{os.path.abspath(app)}:/app.conf", "-v", f"{os.path.abspath(data)}:/data",
              "-v", f"{os.path.abspath(model)}:/model"]
    sched = node_string("SCHEDULER", ip, port, "H")
    args = ["-app_file", "/app.conf", "-num_servers", str(num_servers), "-num_workers", str(num_workers)] + list(extra)
    cmds = []
    for i in range(num_servers + num_workers + 1):
        p = port + i
        if i == 0:
            node = sched
        elif i <= num_servers:
            node = node_string("SERVER", ip, p, f"S{i - 1}")
        else:
            node = node_string("WORKER", ip, p, f"W{i - num_servers - 1}")
        cmds.append(["docker", "run", "--rm", "-p", f"{p}:{p}", "--name", f"n{i}", *mounts, image, BIN_IN_IMAGE,
                     "-my_node", node, "-scheduler", sched, *args])
    return cmds


def upload_command(local_file: str, s3_path: str) -> List[str]:
    """`curl --upload-file` of one file to a public-read S3 object, the job of ``docker/upload_s3.sh:1-24``
    (data or a configuration that the containers then read as ``s3://bucket/key``)."""
    if not s3_path.startswith("s3://") or "/" not in s3_path[5:]:
        raise SystemExit("upload: the target must be s3://bucket/key")
    bucket, key = s3_path[5:].split("/", 1)
    size = os.path.getsize(local_file)
    return ["curl", f"http://{bucket}.s3.amazonaws.com/{key}?Content-Length={size}&x-amz-acl=public-read",
            "--upload-file", local_file]


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    dry = "--dry-run" in argv
    argv = [a for a in argv if a != "--dry-run"]
    image = IMAGE
    if "-image" in argv:
        k = argv.index("-image")
        image = argv[k + 1]
        del argv[k:k + 2]
    if not argv:
        print(__doc__)
        return 2
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if argv[0] == "build":
        cmds = [["docker", "build", "-t", image, "-f", os.path.join(root, "docker", "Dockerfile"), root]]
    elif argv[0] == "local" and len(argv) >= 6:
        cmds = local_commands(int(argv[1]), int(argv[2]), argv[3], argv[4], argv[5], argv[6:], bridge_ip(), image)
    elif argv[0] == "rm" and len(argv) >= 3:
        cmds = [["docker", "rm", "-f"] + [f"n{i}" for i in range(int(argv[1]) + int(argv[2]) + 1)]]
    elif argv[0] == "upload" and len(argv) == 3:
        cmds = [upload_command(argv[1], argv[2])]
    else:
        print(__doc__)
        return 2
    if dry:
        for c in cmds:
            print(" ".join(shlex.quote(x) for x in c))
        return 0
    procs = [subprocess.Popen(c) for c in cmds]
    return max((p.wait() for p in procs), default=0)


if __name__ == "__main__":
    sys.exit(main())
