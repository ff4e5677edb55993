"""Device KVMap / KVVector Push/Pull API: timestamps, wait dependencies, callbacks."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_kv_vector_push_pull_timestamps_and_callbacks(cuda_lib, tmp_path):
    from parameter_server_b200.parameter.kv import DeviceKVVector
    kv = DeviceKVVector.create(table_capacity=1 << 12, max_keys=1 << 10)
    keys = np.array([3, 17, 1 << 40, (1 << 63) + 5], dtype=np.uint64)
    called = []
    t0 = kv.push(keys, [1.0, 2.0, 3.0, 4.0])
    t1 = kv.push(keys[1:3], [10.0, 20.0], callback=lambda: called.append("p1"))
    t2 = kv.pull(keys, wait=[t1], callback=lambda: called.append("pull"))
    assert (t0, t1, t2) == (0, 1, 2)
    kv.wait(t1); kv.wait(t2)
    assert called == ["p1", "pull"]
    assert kv.result(t2).cpu().tolist() == [1.0, 12.0, 23.0, 4.0]
    t3 = kv.pull(np.array([5, 17], dtype=np.uint64), ts=10)        # explicit timestamp, an absent key reads 0
    assert t3 == 10 and kv.pull(keys[:1]) == 11
    kv.wait(10)
    assert kv.result(10).cpu().tolist() == [0.0, 12.0]
    kv.write_to_file(str(tmp_path / "dump_S0"))
    lines = open(tmp_path / "dump_S0").read().splitlines()
    assert lines[0] == "3\t1" and lines[1] == "17\t12" and len(lines) == 4


def test_kv_map_ftrl_entries(cuda_lib):
    from parameter_server_b200.parallel.dataplane import OptimizerConfig
    from parameter_server_b200.parameter.kv import DeviceKVMap
    from parameter_server_b200.utils import oracle
    opt = OptimizerConfig(algo="ftrl", alpha=0.1, beta=1.0, l1=0.01, l2=0.1)
    kv = DeviceKVMap.create(table_capacity=1 << 12, max_keys=1 << 10, opt=opt)
    ot = oracle.OracleTable(opt)
    rng = np.random.default_rng(0)
    universe = np.unique(rng.integers(0, 1 << 62, 200, dtype=np.uint64))
    for _ in range(5):
        k = np.sort(rng.choice(universe, 50, replace=False))
        g = rng.normal(size=50).astype(np.float32)
        kv.push(k, g)
        ot.push(k, g)
    ts = kv.pull(universe)
    kv.wait(ts)
    assert np.allclose(kv.result(ts).cpu().numpy(), ot.pull(universe), rtol=1e-4, atol=1e-6)
