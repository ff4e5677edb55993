"""GPU ranks as parameter-server nodes: the control flow (scheduler, workload pool, round
leases, progress, model dump, lost nodes) on CPU processes with a counting engine."""
import os
import signal
import subprocess
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write_files(d, sizes, seed=0):
    rng = np.random.default_rng(seed)
    files = []
    for f, n in enumerate(sizes):
        p = os.path.join(d, f"part-{f:02d}")
        with open(p, "w") as out:
            for _ in range(n):
                idx = sorted(set(rng.integers(1, 1000, 8).tolist()))
                out.write(("1" if rng.random() < 0.5 else "-1") + " " + " ".join(f"{j}:1" for j in idx) + "\n")
        files.append(p)
    return files


def _conf(d, minibatch=50, passes=1):
    p = os.path.join(d, "job.conf")
    with open(p, "w") as f:
        f.write(f'''training_data {{ format: TEXT text: LIBSVM file: "{d}/part-.*" }}
model_output {{ format: TEXT file: "{d}/model" }}
loss {{ type: LOGIT }}
penalty {{ type: L1 lambda: 1 }}
learning_rate {{ type: DECAY alpha: 0.1 beta: 1 }}
async_sgd {{ algo: FTRL minibatch: {minibatch} num_data_pass: {passes} report_interval: 0.05 }}
''')
    return p


def test_single_process_job(tmp_path):
    from parameter_server_b200.app import nodes as N
    d = str(tmp_path)
    files = _write_files(d, [230, 240, 250, 260, 270])
    eng = N.NullEngine()
    rn = N.start_rank_nodes(0, 1, N.scheduler_spec("inproc", 31000), files=files, passes=2, lease=16, inproc=True)
    res = N.run_lockstep_worker_loop(rn, eng, minibatch=50, model_file=os.path.join(d, "model"), report_interval=0.02)
    assert res["examples"] == 2 * sum([230, 240, 250, 260, 270]) and res["files"] == 10
    assert res["rounds"] == eng.rounds == rn.scheduler.round_limit()      # stopped exactly at the final limit
    assert rn.scheduler.num_finished() == rn.scheduler.num_workloads() == 10
    assert eng.saved == [os.path.join(d, "model_S0")]


def _launch(d, conf, n_procs, roles, n_servers, n_workers, step_seconds=0.0, port=None):
    from parameter_server_b200.app import nodes as N
    from parameter_server_b200.system import core
    spec = N.scheduler_spec("127.0.0.1", port or core.free_port())
    procs = []
    for r in range(n_procs):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(n_procs), PSB_SCHEDULER=spec, PSB_ROLES=roles[r],
                   PSB_NUM_SERVERS=str(n_servers), PSB_NUM_WORKERS=str(n_workers), PSB_ROUND_LEASE="16",
                   PSB_NULL_STEP_SECONDS=str(step_seconds), PYTHONPATH=ROOT)
        procs.append(subprocess.Popen([sys.executable, "-m", "parameter_server_b200.app.linear", "-app_file", conf,
                                       "-engine", "null"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                      text=True, cwd=ROOT))
    return procs


def _summary(out):
    for line in out.splitlines():
        if "] rounds " in line:
            a = line.split()
            return int(a[a.index("rounds") + 1]), int(a[a.index("examples") + 1]), int(a[a.index("files") + 1])
    raise AssertionError("no summary line in:\n" + out)


def test_three_processes_uneven_files(tmp_path):
    """Seven files of different sizes over three ranks: files are handed out one at a time, every rank
    runs the same number of rounds (ranks without data run empty rounds) and stops at the same one."""
    d = str(tmp_path)
    sizes = [400, 90, 60, 310, 45, 120, 75]
    _write_files(d, sizes)
    conf = _conf(d)
    procs = _launch(d, conf, 3, ["HSW", "SW", "SW"], 3, 3, step_seconds=0.002)
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    res = [_summary(o) for o in outs]
    assert len({r[0] for r in res}) == 1, res                  # same final round everywhere
    assert sum(r[1] for r in res) == sum(sizes) and sum(r[2] for r in res) == len(sizes)
    assert all(os.path.exists(os.path.join(d, f"model_S{r}")) for r in range(3))
    assert "examples" in outs[0] and "loss" in outs[0]         # the scheduler's progress table


def test_worker_killed_between_steps_files_requeued(tmp_path):
    """A worker process is killed in mid-run: the scheduler's manager notices the lost connection, puts
    the worker's unfinished file back into the pool and hands it to a worker that had run out of work;
    the survivors learn of the lost node (REMOVE_NODE) and mark its rank dead in their engine."""
    d = str(tmp_path)
    sizes = [300, 300, 300, 300, 300, 300]
    _write_files(d, sizes)
    conf = _conf(d, minibatch=20)
    # rank 2 hosts a worker only (no key-range shard is lost with it)
    procs = _launch(d, conf, 3, ["HSW", "SW", "W"], 2, 3, step_seconds=0.01)
    # wait until the worker has a file, let it run a few minibatches, then kill it
    t0 = time.time()
    while True:
        line = procs[2].stdout.readline()
        assert line and time.time() - t0 < 120, "worker 2 never started"
        if "first workload" in line:
            break
    time.sleep(0.1)
    procs[2].send_signal(signal.SIGKILL)
    outs = [p.communicate(timeout=180)[0] for p in procs[:2]]
    procs[2].communicate()
    assert all(p.returncode == 0 for p in procs[:2]), "\n".join(outs)
    res = [_summary(o) for o in outs]
    assert res[0][0] == res[1][0]
    # every file was finished by a survivor or, before it died, by the lost worker
    assert sum(r[2] for r in res) >= len(sizes) - 2 and sum(r[1] for r in res) >= sum(sizes) - 2 * 300
    for o in outs:
        assert "node W2 lost" in o, o


def test_tail_feature_filter_of_the_loader():
    """async_sgd.tail_feature_freq in the GPU application: a feature's nonzeros pass once the count-min
    estimate of its count so far exceeds the threshold; rows keep their places."""
    import numpy as np
    from parameter_server_b200.app.nodes import TailFeatureFilter
    f = TailFeatureFilter(freq=2, countmin_n=1 << 16, countmin_k=2)

    def batch(rows):
        off = np.cumsum([0] + [len(r) for r in rows]).astype(np.uint64)
        idx = np.array([k for r in rows for k in r], dtype=np.uint64)
        return np.ones(len(rows), np.float32), [dict(id=1, offset=off, index=idx, value=np.arange(len(idx), dtype=np.float32), binary=False)]

    # key 5 appears three times in the first minibatch (kept at once), key 9 twice, key 11 once
    y, (m,) = f.apply(batch([[5, 9], [5, 11], [5, 9]]))
    assert list(m["offset"]) == [0, 1, 2, 3] and list(m["index"]) == [5, 5, 5] and list(m["value"]) == [0, 2, 4]
    # second minibatch: 9 has now been seen three times, 11 twice
    y, (m,) = f.apply(batch([[9], [11], []]))
    assert list(m["offset"]) == [0, 1, 1, 1] and list(m["index"]) == [9]
    y, (m,) = f.apply(batch([[11, 5]]))
    assert list(m["index"]) == [11, 5] and f.dropped == 4


def test_application_reads_tail_filter_from_the_configuration(tmp_path):
    """The application (node layer only, counting engine) runs a job whose async_sgd block sets the filter."""
    d = str(tmp_path)
    _write_files(d, [120, 130])
    conf = _conf(d, minibatch=50)
    text = open(conf).read().replace("report_interval: 0.05", "report_interval: 0.05 tail_feature_freq: 2 countmin_n: 65536")
    open(conf, "w").write(text)
    procs = _launch(d, conf, 1, ["HSW"], 1, 1)
    out = procs[0].communicate(timeout=120)[0]
    assert procs[0].returncode == 0, out[-2000:]
    assert _summary(out)[1:] == (250, 2)


def test_application_reads_binary_matrices(tmp_path):
    """format: BIN in the data section: one workload per matrix (not per companion file), minibatches are slices
    of the mapped files (node layer with the counting engine)."""
    from parameter_server_b200.utils import datatool
    d = str(tmp_path)
    _write_files(d, [120, 130])
    for i in range(2):
        assert datatool.main(["convert", "-input", f"{d}/part-0{i}", "-output", f"{d}/bin-{i}", "-to", "bin"]) == 0
    conf = _conf(d, minibatch=50)
    text = open(conf).read().replace('format: TEXT text: LIBSVM file: "%s/part-.*"' % d, 'format: BIN file: "%s/bin-.*"' % d)
    assert "format: BIN" in text
    open(conf, "w").write(text)
    procs = _launch(d, conf, 1, ["HSW"], 1, 1)
    out = procs[0].communicate(timeout=120)[0]
    assert procs[0].returncode == 0, out[-2000:]
    assert _summary(out)[1:] == (250, 2)
