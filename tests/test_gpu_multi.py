"""Real multi-GPU run of the data plane: one process per GPU, heaps mapped over
CUDA IPC, peer loads/stores over NVLink. Skipped with fewer than two GPUs.

The ranks run ``python -m parameter_server_b200.parallel.selftest`` under
``torch.distributed.run``; the result is compared with the CPU oracle there.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("quant,pull,tau", [("none", "exchange", 0), ("none", "exchange", 2), ("int8", "exchange", 0),
                                            ("none", "one-sided", 0), ("none", "one-sided", 1)])
def test_two_rank_training_matches_oracle(cuda_lib, quant, pull, tau):
    """tau = 0 is compared tightly with the sequential oracle; with tau > 0 a pull may
    see a model that is up to tau rounds old, so only rough agreement is required."""
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29731", "-m",
           "parameter_server_b200.parallel.selftest", "--quant", quant, "--pull", pull, "--tau", str(tau)]
    r = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "SELFTEST OK" in r.stdout


@pytest.mark.parametrize("what", ["layer", "kv", "darlin", "wide"])
def test_other_planes_over_real_peers(cuda_lib, what):
    """KVLayer (back-to-back rounds, no host barrier), the KV containers, Darlin and the wide-value
    exchange pull (single cooperative launch, all roles) over real peer mappings."""
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29751", "-m",
           "parameter_server_b200.parallel.selftest_peers", "--what", what]
    r = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "SELFTEST OK" in r.stdout


APP_CONF = """
training_data {{ format: TEXT text: SPARSE_BINARY file: "{train}/part.*" }}
model_output {{ format: TEXT file: "{out}/model" }}
loss {{ type: LOGIT }}
penalty {{ type: L1 lambda: 0.5 lambda: 0.01 }}
learning_rate {{ type: DECAY alpha: 0.1 beta: 1 }}
async_sgd {{ algo: FTRL minibatch: 500 num_data_pass: 2 max_delay: 1 report_interval: 0.2 }}
"""


def test_two_rank_app_is_a_parameter_server_job(cuda_lib, tmp_path):
    """``app.linear`` under torch.distributed.run: every rank hosts a server and a worker node, rank 0
    the scheduler; three files of different sizes over two ranks (dynamic assignment, empty rounds
    for the rank without data), progress table from the scheduler's monitor, one model file per
    server; the model evaluates like a single-GPU one."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    from parameter_server_b200.app import linear
    from parameter_server_b200.system import core
    from parameter_server_b200.utils.textdata import write_sparse_binary
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    write_sparse_binary(str(tmp_path / "train"), 3, 1500, 12, 400, seed=1)
    # make the files uneven: drop two thirds of the last one
    last = sorted((tmp_path / "train").glob("part*"))[-1]
    lines = last.read_text().splitlines()
    last.write_text("\n".join(lines[:500]) + "\n")
    conf = tmp_path / "job.conf"
    conf.write_text(APP_CONF.format(train=tmp_path / "train", out=tmp_path))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root, PSB_LOG2_TABLE="14", PSB_MAX_NNZ_PER_ROW="16")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29741", "-m",
           "parameter_server_b200.app.linear", "-app_file", str(conf)]
    r = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    out = r.stdout + r.stderr
    rounds = [int(l.split("rounds")[1].split()[0]) for l in out.splitlines() if "] rounds " in l]
    examples = [int(l.split("examples")[1].split()[0]) for l in out.splitlines() if "] rounds " in l]
    assert len(rounds) == 2 and rounds[0] == rounds[1], out[-2000:]
    assert sum(examples) == 2 * (1500 + 1500 + 500)
    assert (tmp_path / "model_S0").exists() and (tmp_path / "model_S1").exists()
    ev = linear.run_evaluation(core.parse_text_proto(
        f'validation_data {{ format: TEXT text: SPARSE_BINARY file: "{tmp_path}/train/part.*" }}\n'
        f'model_input {{ format: TEXT file: "{tmp_path}/model_S.*" }}'), verbose=False)
    assert ev["auc"] > 0.68 and ev["logloss"] < 0.67
