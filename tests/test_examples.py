"""The tutorial under examples/linear runs as written: data generator, online and batch training and the
two evaluations with the shipped configuration files, CPU nodes as local processes."""
import glob
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CONF = os.path.join(ROOT, "examples", "linear", "ctr")


def _run(conf, ns, nw):
    from parameter_server_b200 import _build
    from parameter_server_b200.system.cluster import launch_local_processes
    _build.build_core()
    exe = os.path.join(ROOT, "parameter_server_b200", "bin", "psb_linear")
    out = launch_local_processes(ns, nw, [exe, "-app_file", os.path.join(CONF, conf)], timeout=240)
    assert all(p.returncode == 0 for p in out.values()), {k: (p.returncode, p.stdout[-400:]) for k, p in out.items()}
    return out["H"].stdout


def test_tutorial_configs_train_and_evaluate(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    os.makedirs("model")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "linear", "make_data.py"), "--files", "2",
                        "--rows", "2500", "--nnz", "16", "--features", "2000"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert len(glob.glob("data/ctr/train/part-*")) == 2 and len(glob.glob("data/ctr/test/part-*")) == 1
    _run("online_l1lr.conf", 2, 2)
    assert len(glob.glob("model/ctr_online_S*")) == 2
    ev = _run("eval_online.conf", 1, 1)
    auc = float(re.search(r"auc[:= ]+([0-9.]+)", ev, re.I).group(1))
    assert auc > 0.6, ev[-500:]
    _run("batch_l1lr.conf", 2, 2)
    assert len(glob.glob("model/ctr_batch_S*")) == 2
    ev = _run("eval_batch.conf", 1, 1)
    assert float(re.search(r"auc[:= ]+([0-9.]+)", ev, re.I).group(1)) > 0.6, ev[-500:]


def test_libsvm_and_criteo_examples(tmp_path, monkeypatch):
    """The rcv1-style (LIBSVM, real values) and criteo-style (click-log lines, one feature group per field)
    configurations train and evaluate on generated data of their formats."""
    global CONF
    monkeypatch.chdir(tmp_path)
    os.makedirs("model")
    gen = os.path.join(ROOT, "examples", "linear", "make_data.py")
    for fmt, out in (("libsvm", "data/rcv1"), ("criteo", "data/criteo")):
        r = subprocess.run([sys.executable, gen, "--format", fmt, "--out", out, "--files", "2", "--rows", "2000", "--nnz", "16",
                            "--features", "2000"], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    keep = CONF
    try:
        CONF = os.path.join(ROOT, "examples", "linear", "rcv1")
        _run("online_l1lr.conf", 2, 2)
        assert float(re.search(r"auc[:= ]+([0-9.]+)", _run("eval_online.conf", 1, 1), re.I).group(1)) > 0.6
        _run("batch_l1lr.conf", 2, 2)
        assert float(re.search(r"auc[:= ]+([0-9.]+)", _run("eval_batch.conf", 1, 1), re.I).group(1)) > 0.6
        CONF = os.path.join(ROOT, "examples", "linear", "criteo")
        _run("batch_l1lr.conf", 2, 2)
        assert float(re.search(r"auc[:= ]+([0-9.]+)", _run("eval_batch.conf", 1, 1), re.I).group(1)) > 0.6
    finally:
        CONF = keep


def test_kv_api_examples():
    """The two small programs under examples/kv run as a user would run them."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "examples", "kv", "hello.py")],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert out.stdout.count("hello world") == 3 and "every server has answered" in out.stdout
    assert "last response came from S1" in out.stdout
    out = subprocess.run([sys.executable, os.path.join(root, "examples", "kv", "kv_vector.py")],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert "pulled [3.0, 6.0, 9.0]" in out.stdout
    out = subprocess.run([sys.executable, os.path.join(root, "examples", "kv", "kv_layer.py")],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert "layer 2: 1000 values, every one 3" in out.stdout and "held as [500, 500]" in out.stdout


def test_cpp_programs_link_static_runtime(tmp_path):
    """C++ programs link against lib/libpsb.a (and lib/libpsbmain.a when they define only CreateServerNode /
    WorkerNodeMain) and run as scheduler + 2 servers + 2 workers over TCP."""
    from parameter_server_b200 import _build
    from parameter_server_b200.system.cluster import launch_local_processes
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib, main_lib = _build.build_static()
    cxx = os.environ.get("PSB_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")

    def compile_(name, libs):
        exe = tmp_path / name
        subprocess.run([cxx, "-O1", "-std=c++17", "-pthread", "-I", os.path.join(root, "parameter_server_b200", "csrc", "core"),
                        os.path.join(root, "examples", "cpp", name + ".cc"), *map(str, libs), "-lz", "-o", str(exe)],
                       check=True, timeout=600)
        return str(exe)

    out = launch_local_processes(2, 2, [compile_("kv_sum", [main_lib, lib])], timeout=120)
    assert all(p.returncode == 0 for p in out.values()), {k: (p.returncode, p.stdout[-300:]) for k, p in out.items()}
    for w in ("W0", "W1"):
        assert f"{w} pulled 3 6 9" in out[w].stdout
    out = launch_local_processes(1, 2, [compile_("aggregation", [lib])], timeout=120)
    assert all(p.returncode == 0 for p in out.values()), {k: (p.returncode, p.stdout[-300:]) for k, p in out.items()}
    assert "W0 pulled 8 12 8 12 8 12 4 6" in out["W0"].stdout and "W1 pulled 8 12 4 6 8 12 8 12" in out["W1"].stdout
    out = launch_local_processes(2, 2, [compile_("network_perf", [lib]), "-n=20", "-data_size=200"], timeout=120)
    assert all(p.returncode == 0 for p in out.values()), {k: (p.returncode, p.stdout[-300:]) for k, p in out.items()}
    for w in ("W0", "W1"):
        m = re.search(r"packet size 200 KB to 2 servers, 20 rounds, throughput ([0-9.]+) MB/s", out[w].stdout)
        assert m and float(m.group(1)) > 1.0, out[w].stdout
