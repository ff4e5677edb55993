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
