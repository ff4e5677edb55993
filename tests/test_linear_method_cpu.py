"""CPU linear-method applications end to end: async SGD (FTRL / AdaGrad) and
Darlin, in-process and as real OS processes over TCP (the counterpart of
`script/local.sh 2 2 build/linear -app_file ...`), plus model evaluation."""
import glob
import os
import sys

import numpy as np
import pytest

from parameter_server_b200.system import LocalCluster, core
from parameter_server_b200.system.cluster import launch_local_processes
from parameter_server_b200.utils.textdata import key_of_id, write_sparse_binary

CONF_SGD = """
training_data {{ format: TEXT text: SPARSE_BINARY file: "{train}/part.*" }}
model_output {{ format: TEXT file: "{out}/model" }}
loss {{ type: LOGIT }}
penalty {{ type: L1 lambda: 0.5 lambda: 0.01 }}
learning_rate {{ type: DECAY alpha: 0.1 beta: 1 }}
async_sgd {{
  algo: {algo}
  ada_grad: true
  minibatch: 500
  num_data_pass: 3
  max_delay: 2
  {filters}
}}
"""

FILTERS = """
  push_filter { type: KEY_CACHING clear_cache_if_done: true }
  push_filter { type: FIXING_FLOAT num_bytes: 2 }
  pull_filter { type: KEY_CACHING }
  pull_filter { type: COMPRESSING }
"""

CONF_EVAL = """
validation_data {{ format: TEXT text: SPARSE_BINARY file: "{val}/part.*" }}
model_input {{ format: TEXT file: "{out}/model_S.*" }}
"""

CONF_DARLIN = """
training_data {{ format: TEXT text: SPARSE_BINARY file: "{train}/part.*" }}
model_output {{ format: TEXT file: "{out}/darlin" }}
loss {{ type: LOGIT }}
penalty {{ type: L1 lambda: 2 }}
learning_rate {{ type: CONSTANT alpha: 0.5 }}
darlin {{
  max_pass_of_data: 12
  epsilon: 1e-4
  max_block_delay: {tau}
  feature_block_ratio: 0.4
  tail_feature_freq: {tail}
  comm_filter {{ type: KEY_CACHING }}
}}
"""


def _read_model(pattern):
    w = {}
    for f in glob.glob(pattern):
        for line in open(f):
            k, v = line.split("\t")
            w[int(k)] = float(v)
    return w


def _score(files, w):
    y, m = [], []
    for f in files:
        for line in open(f):
            parts = line.strip().split(";")
            y.append(float(parts[0]))
            m.append(sum(w.get(int(k), 0.0) for k in parts[1].split()[1:]))
    return np.array(y, np.float32), np.array(m, np.float32)


@pytest.fixture(scope="module")
def data(tmp_path_factory):
    root = tmp_path_factory.mktemp("lm")
    train, _ = write_sparse_binary(str(root / "train"), 4, 1500, 12, 400, seed=1)
    val, _ = write_sparse_binary(str(root / "val"), 1, 1500, 12, 400, seed=1, prefix="part-val")
    # same ground truth for validation: regenerate with the same seed, but skip the training rows
    return dict(root=str(root), train=str(root / "train"), val=str(root / "val"), train_files=train, val_files=val)


@pytest.mark.parametrize("algo,filters", [("FTRL", ""), ("FTRL", FILTERS), ("STANDARD", "")])
def test_async_sgd_in_process(data, tmp_path, algo, filters):
    conf = CONF_SGD.format(train=data["train"], out=str(tmp_path), algo=algo, filters=filters)
    cl = LocalCluster(2, 2, None, conf=conf, run=True)
    cl.join(timeout=120)
    cl.stop()
    w = _read_model(str(tmp_path / "model_S*"))
    assert len(w) > 10
    y, m = _score(data["train_files"], w)
    ev = core.evaluate(y, m)
    assert ev["auc"] > 0.68 and ev["logloss"] < 0.67, ev
    # shards hold disjoint key ranges
    s0 = set(_read_model(str(tmp_path / "model_S0"))); s1 = set(_read_model(str(tmp_path / "model_S1")))
    assert s0 and s1 and not (s0 & s1)
    # ranks follow registration order, so either server may own the lower half
    halves = sorted([(min(s0), max(s0)), (min(s1), max(s1))])
    assert halves[0][1] < (1 << 63) <= halves[1][0]


def test_model_evaluation_app(data, tmp_path):
    conf = CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters="")
    cl = LocalCluster(1, 1, None, conf=conf, run=True)
    cl.join(timeout=120)
    cl.stop()
    ev = LocalCluster(0, 0, None, conf=CONF_EVAL.format(val=data["train"], out=str(tmp_path)), run=True)
    ev.join(timeout=60)
    ev.stop()


@pytest.mark.parametrize("tau,tail", [(0, 0), (2, 0), (1, 2)])
def test_darlin_in_process(data, tmp_path, tau, tail):
    conf = CONF_DARLIN.format(train=data["train"], out=str(tmp_path), tau=tau, tail=tail)
    cl = LocalCluster(2, 2, None, conf=conf, run=True)
    cl.join(timeout=180)
    cl.stop()
    w = _read_model(str(tmp_path / "darlin_S*"))
    assert 5 < len(w) < 400
    y, m = _score(data["train_files"], w)
    ev = core.evaluate(y, m)
    # with a delay the few, strongly coupled blocks of this small problem converge more slowly
    assert ev["auc"] > (0.68 if tau == 0 else 0.64), ev
    # objective of the dumped model: logistic loss + lambda |w|_1 must beat the zero model
    obj = np.log1p(np.exp(-y * m)).sum() + 2 * sum(abs(v) for v in w.values())
    assert obj < (0.93 if tau == 0 else 0.99) * len(y) * np.log(2)


def test_darlin_starts_from_given_weights(data, tmp_path):
    """darlin { init_w { type: CONSTANT constant: c } }: the servers allocate the weights with that value and the
    workers start from dual = exp(y . Xw). After one pass the model differs from the zero start's; after twelve
    it has reached the same neighbourhood of the optimum of this convex problem."""
    const = "init_w { type: CONSTANT constant: 0.05 }"
    objs = {}
    for name, init, passes in (("zero", "", 12), ("const", const, 12), ("zero1", "", 1), ("const1", const, 1)):
        out = tmp_path / name
        out.mkdir()
        conf = CONF_DARLIN.format(train=data["train"], out=str(out), tau=0, tail=0).replace(
            "max_pass_of_data: 12", f"max_pass_of_data: {passes} random_feature_block_order: false {init}")
        cl = LocalCluster(2, 2, None, conf=conf, run=True)
        cl.join(timeout=180)
        cl.stop()
        w = _read_model(str(out / "darlin_S*"))
        y, m = _score(data["train_files"], w)
        objs[name] = (np.log1p(np.exp(-y * m)).sum() + 2 * sum(abs(v) for v in w.values()), w)
    assert objs["const1"][1] != objs["zero1"][1]
    assert objs["const"][0] < 0.95 * len(y) * np.log(2)          # well below the zero model
    assert abs(objs["const"][0] - objs["zero"][0]) < 0.1 * objs["zero"][0], (objs["const"][0], objs["zero"][0])


def test_async_sgd_multi_process_tcp(data, tmp_path):
    """1 scheduler + 2 servers + 2 workers as OS processes on 127.0.0.1."""
    from parameter_server_b200 import _build
    exe = str(_build.PKG / "bin" / "psb_linear")
    conf = tmp_path / "sgd.conf"
    conf.write_text(CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters=FILTERS))
    res = launch_local_processes(2, 2, [exe, "-app_file", str(conf)], timeout=180)
    for nid, r in res.items():
        assert r.returncode == 0, (nid, r.stdout[-2000:])
    assert "examples" in res["H"].stdout          # the scheduler printed the progress table
    w = _read_model(str(tmp_path / "model_S*"))
    y, m = _score(data["train_files"], w)
    assert core.evaluate(y, m)["auc"] > 0.68


@pytest.mark.parametrize("kinds", ["address,undefined", "thread"])
def test_node_processes_clean_under_sanitizers(data, tmp_path, kinds):
    """The stand-alone node binary built with -fsanitize=<kinds> runs async SGD (with
    the filter chain) and Darlin as 1 scheduler + 2 servers + 2 workers over TCP
    without a single sanitizer report (memory errors, undefined behaviour, data races)."""
    from parameter_server_b200 import _build
    exe = str(_build.build_sanitized_binary(kinds))
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=0", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1",
               TSAN_OPTIONS="halt_on_error=0")
    confs = {"sgd": CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters=FILTERS),
             "darlin": CONF_DARLIN.format(train=data["train"], out=str(tmp_path), tau=1, tail=2)}
    for name, text in confs.items():
        conf = tmp_path / f"{name}.conf"
        conf.write_text(text)
        res = launch_local_processes(2, 2, [exe, "-app_file", str(conf)], timeout=120, env=env)
        for nid, r in res.items():
            out = r.stdout or ""
            assert r.returncode == 0, (name, nid, out[-3000:])
            assert "Sanitizer" not in out and "runtime error" not in out, (name, nid, out[-3000:])
    assert len(_read_model(str(tmp_path / "model_S*"))) > 10


def test_training_data_in_hdfs(data, tmp_path):
    """training_data with an `hdfs` block: scheduler and workers (OS processes) list and read the files through
    `<home>/bin/hadoop fs` (a stand-in command that serves local files), for the online and the batch solver."""
    from test_core_util import _fake_hadoop
    from parameter_server_b200 import _build
    log = tmp_path / "hadoop.log"
    _fake_hadoop(tmp_path / "hadoop", log)
    exe = str(_build.PKG / "bin" / "psb_linear")
    hdfs = f'hdfs {{ home: "{tmp_path}/hadoop" namenode: "nn:9000" }} file:'
    for name, text in (("sgd", CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters="")),
                       ("darlin", CONF_DARLIN.format(train=data["train"], out=str(tmp_path), tau=1, tail=0))):
        conf = tmp_path / f"{name}.conf"
        conf.write_text(text.replace("file:", hdfs, 1))
        assert "hdfs {" in conf.read_text().splitlines()[1]
        res = launch_local_processes(2, 2, [exe, "-app_file", str(conf)], timeout=180)
        for nid, r in res.items():
            assert r.returncode == 0, (name, nid, r.stdout[-2000:])
    calls = log.read_text()
    assert f"-ls hdfs://{data['train']}" in calls and f"-cat hdfs://{data['train']}/part-" in calls
    w = _read_model(str(tmp_path / "model_S*"))
    y, m = _score(data["train_files"], w)
    assert core.evaluate(y, m)["auc"] > 0.68
    assert len(_read_model(str(tmp_path / "darlin_S*"))) > 10


def test_reader_flags_on_the_command_line(data, tmp_path):
    """-hash_kernel N folds every feature id into [0, N) in the stream reader; -line_limit caps the lines read
    per text file (the reference's global flags of the same names)."""
    from parameter_server_b200 import _build
    exe = str(_build.PKG / "bin" / "psb_linear")
    conf = tmp_path / "sgd.conf"
    conf.write_text(CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters="")
                    .replace("lambda: 0.5", "lambda: 0.01"))
    res = launch_local_processes(1, 2, [exe, "-app_file", str(conf), "-hash_kernel", "50", "-line_limit=200"], timeout=180)
    for nid, r in res.items():
        assert r.returncode == 0, (nid, r.stdout[-2000:])
    w = _read_model(str(tmp_path / "model_S*"))
    assert 5 < len(w) <= 50 and max(w) < 50
    # the batch solver reads its files line by line: 4 files x 200 lines, not the 1500 lines per file that are there
    conf.write_text(CONF_DARLIN.format(train=data["train"], out=str(tmp_path), tau=0, tail=0))
    res = launch_local_processes(1, 2, [exe, "-app_file", str(conf), "-line_limit=200"], timeout=180)
    for nid, r in res.items():
        assert r.returncode == 0, (nid, r.stdout[-2000:])
    assert "loaded 800 examples" in res["H"].stdout, res["H"].stdout[:600]


def test_training_data_as_binary_matrices(data, tmp_path):
    """format: BIN: the text files converted to binary matrices train the same model family (CPU nodes as OS
    processes); one workload per matrix."""
    from parameter_server_b200 import _build
    from parameter_server_b200.utils import datatool
    bindir = tmp_path / "bin"
    bindir.mkdir()
    for i, f in enumerate(data["train_files"]):
        assert datatool.main(["convert", "-input", f, "-output", str(bindir / f"part-{i}"), "-format", "sparse_binary", "-to", "bin"]) == 0
    conf = tmp_path / "sgd.conf"
    conf.write_text(CONF_SGD.format(train=str(bindir), out=str(tmp_path), algo="FTRL", filters="")
                    .replace("format: TEXT text: SPARSE_BINARY", "format: BIN", 1))
    res = launch_local_processes(2, 2, [str(_build.PKG / "bin" / "psb_linear"), "-app_file", str(conf)], timeout=180)
    for nid, r in res.items():
        assert r.returncode == 0, (nid, r.stdout[-2000:])
    w = _read_model(str(tmp_path / "model_S*"))
    y, m = _score(data["train_files"], w)
    assert core.evaluate(y, m)["auc"] > 0.68


def test_scheduler_only_job_waits_for_late_nodes(data, tmp_path):
    """Model evaluation is done by the scheduler alone and takes milliseconds here; a server and a worker that
    start a second later must still find the scheduler, register, and be released by the exit handshake."""
    import subprocess
    import time
    from parameter_server_b200 import _build
    from parameter_server_b200.system.cluster import node_string
    exe = str(_build.PKG / "bin" / "psb_linear")
    train = tmp_path / "sgd.conf"
    train.write_text(CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters=""))
    res = launch_local_processes(1, 1, [exe, "-app_file", str(train)], timeout=180)
    assert all(r.returncode == 0 for r in res.values())
    conf = tmp_path / "eval.conf"
    conf.write_text(CONF_EVAL.format(val=data["val"], out=str(tmp_path)))
    sched = node_string("SCHEDULER", "127.0.0.1", core.free_port(), "H")
    procs = {}
    for nid, role, delay in (("H", "SCHEDULER", 0.0), ("S0", "SERVER", 1.0), ("W0", "WORKER", 0.0)):
        time.sleep(delay)
        spec = sched if nid == "H" else node_string(role, "127.0.0.1", core.free_port(), nid)
        procs[nid] = subprocess.Popen([exe, "-app_file", str(conf), "-my_node", spec, "-scheduler", sched,
                                       "-num_servers", "1", "-num_workers", "1"],
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    outs = {nid: p.communicate(timeout=120)[0] for nid, p in procs.items()}
    assert all(p.returncode == 0 for p in procs.values()), {k: (procs[k].returncode, v[-400:]) for k, v in outs.items()}
    assert "auc" in outs["H"].lower()


def test_darlin_processes_start_reliably(data, tmp_path):
    """Twenty start-ups of 1 scheduler + 2 servers + 2 workers as OS processes: every node
    must be a member of the groups before the scheduler's first group task goes out (a node
    used to be counted as ready too early, and about 3 % of the start-ups hung)."""
    from parameter_server_b200 import _build
    exe = str(_build.PKG / "bin" / "psb_linear")
    conf = tmp_path / "darlin.conf"
    conf.write_text(CONF_DARLIN.format(train=data["train"], out=str(tmp_path), tau=1, tail=0))
    for i in range(20):
        res = launch_local_processes(2, 2, [exe, "-app_file", str(conf)], timeout=30)
        for nid, r in res.items():
            assert r.returncode == 0, (i, nid, (r.stdout or "")[-1500:])


def test_job_control_start_ls_kill_add_stop(data, tmp_path):
    """The job-control commands (the reference's script/ps.sh): start a job, list it, kill a
    worker in mid-run (the scheduler re-queues its workloads and the job still finishes),
    and stop a second job by hand."""
    import time
    from parameter_server_b200 import _build
    from parameter_server_b200.system.launch import Job
    exe = str(_build.PKG / "bin" / "psb_linear")
    conf = tmp_path / "sgd.conf"
    conf.write_text(CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters="")
                    .replace("num_data_pass: 3", "num_data_pass: 200"))
    job = Job(str(tmp_path / "state.json"))
    nodes = job.start([exe, "-app_file", str(conf)], num_servers=2, num_workers=2, log_dir=str(tmp_path / "logs"))
    assert [n["id"] for n in nodes] == ["H", "S0", "S1", "W0", "W1"]
    # a second Job object (another invocation of the tool) finds the job through the state file
    seen = Job(str(tmp_path / "state.json")).ls()
    assert len(seen) == 5 and all(n["alive"] for n in seen)
    time.sleep(0.3)
    assert job.kill("W1")                       # a worker dies in mid-run
    assert job.wait(120), [open(n["log"]).read()[-800:] for n in job.ls() if n["alive"]]
    sched_log = open(nodes[0]["log"]).read()
    assert "examples" in sched_log              # the scheduler printed its progress table
    assert len(_read_model(str(tmp_path / "model_S*"))) > 10
    job.stop()
    assert not os.path.exists(str(tmp_path / "state.json"))
    # stop: a long job is ended by hand
    conf.write_text(conf.read_text().replace("num_data_pass: 200", "num_data_pass: 100000"))
    job = Job(str(tmp_path / "state.json"))
    job.start([exe, "-app_file", str(conf)], num_servers=1, num_workers=1, log_dir=str(tmp_path / "logs2"))
    time.sleep(0.5)
    assert all(n["alive"] for n in job.ls())
    # add: a worker joins the running job through the scheduler's registration path
    assert [n["id"] for n in job.add(workers=1)] == ["W1"]
    time.sleep(0.7)
    assert [n["id"] for n in job.ls() if n["alive"]] == ["H", "S0", "W0", "W1"]
    assert "error" not in open(job.ls()[-1]["log"]).read().lower()
    job.stop()
    assert job.ls() == []


def test_job_control_command_line(data, tmp_path, capsys):
    """The same commands through the module's command line (start -- bin args, ls, wait, stop)."""
    from parameter_server_b200 import _build
    from parameter_server_b200.system import launch
    exe = str(_build.PKG / "bin" / "psb_linear")
    conf = tmp_path / "sgd.conf"
    conf.write_text(CONF_SGD.format(train=data["train"], out=str(tmp_path), algo="FTRL", filters=""))
    st = str(tmp_path / "state.json")
    assert launch.main(["--state", st, "start", "-ns", "1", "-nw", "2", "-log_dir", str(tmp_path / "logs"), "--",
                        exe, "-app_file", str(conf)]) == 0
    assert launch.main(["--state", st, "ls"]) == 0
    out = capsys.readouterr().out
    assert out.count("SERVER") == 2 and out.count("WORKER") == 4 and "SCHEDULER" in out   # start + ls listings
    assert launch.main(["--state", st, "wait", "-timeout", "120"]) == 0
    assert launch.main(["--state", st, "stop"]) == 0
    assert not os.path.exists(st)
    assert len(_read_model(str(tmp_path / "model_S*"))) > 10


def test_job_state_file_is_private_and_pid_reuse_is_harmless(tmp_path, monkeypatch):
    """The job state lives in a 0700 per-user directory; a state file that is not the caller's regular
    file is refused; a recorded pid whose start time no longer matches is never signalled."""
    import os
    import subprocess
    import sys
    from parameter_server_b200.system import launch
    monkeypatch.setenv("XDG_RUNTIME_DIR", str(tmp_path))
    monkeypatch.delenv("PSB_STATE", raising=False)
    p = launch.default_state_path()
    assert p.startswith(str(tmp_path)) and (os.stat(os.path.dirname(p)).st_mode & 0o777) == 0o700
    # a symlink planted at the state path is refused
    target = tmp_path / "elsewhere.json"
    target.write_text("{}")
    os.symlink(target, p)
    with pytest.raises(PermissionError):
        launch.Job()
    os.remove(p)
    # a live process whose recorded start time differs (a recycled pid) counts as gone and is not signalled
    victim = subprocess.Popen([sys.executable, "-c", "import time; time.sleep(30)"], start_new_session=True)
    try:
        job = launch.Job()
        job.state = {"nodes": [{"id": "W0", "pid": victim.pid, "started": (launch._start_time(victim.pid) or 0) + 12345}]}
        assert job.ls()[0]["alive"] is False
        assert job.kill("W0") is False
        job.stop()
        assert victim.poll() is None
        job.state = {"nodes": [{"id": "W0", "pid": victim.pid, "started": launch._start_time(victim.pid)}]}
        assert job.ls()[0]["alive"] is True and job.kill("W0") is True
        victim.wait(10)
    finally:
        if victim.poll() is None:
            victim.kill()
