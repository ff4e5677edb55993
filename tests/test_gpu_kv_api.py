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


def test_key_caching_inside_the_exchange_pull(cuda_lib):
    """A pull with the key list of the previous pull sends no keys: the request areas are poisoned
    after the first pull and the second still answers correctly (the owner used the slots it
    remembered); a different list afterwards is a miss and sends its keys again."""
    from parameter_server_b200.parameter.kv import DeviceKVVector
    kv = DeviceKVVector.create(table_capacity=1 << 14, max_keys=1 << 12, key_cache=True)
    plane = kv.plane
    rng = np.random.default_rng(5)
    keys = np.unique(rng.integers(0, 1 << 62, 3000, dtype=np.uint64))
    vals = rng.normal(size=len(keys)).astype(np.float32)
    kv.push(keys, vals)
    t1 = kv.pull(keys)
    kv.wait(t1)
    assert np.allclose(kv.result(t1).cpu().numpy(), vals)
    req = plane.fabric.view(plane.layout["req_keys"], (2 * plane.S * plane.cfg.inbox_cap,), torch.int64)
    req.fill_(0x1234)
    t2 = kv.pull(keys)                       # same list: a hit, nothing is read from the request areas
    kv.wait(t2)
    assert np.allclose(kv.result(t2).cpu().numpy(), vals)
    assert int((req == 0x1234).all().item()) == 1, "keys were sent although the list did not change"
    other = keys[::3]
    t3 = kv.pull(other)                      # another list: a miss
    kv.wait(t3)
    assert np.allclose(kv.result(t3).cpu().numpy(), vals[::3])
    assert int((req != 0x1234).any().item()) == 1
    t4 = kv.pull(other)                      # and a hit again, right after new values arrived
    kv.push(other, np.ones(len(other), np.float32))
    t5 = kv.pull(other)
    kv.wait(t4); kv.wait(t5)
    assert np.allclose(kv.result(t4).cpu().numpy(), vals[::3])
    assert np.allclose(kv.result(t5).cpu().numpy(), vals[::3] + 1)


@pytest.mark.parametrize("S,k,quant", [(1, 8, "none"), (3, 8, "none"), (2, 64, "none"), (3, 5, "int8")])
def test_kv_vector_of_width_k_with_channels(cuda_lib, S, k, quant):
    """KVVector with k values per key and two channels, on S emulated shards: pushes are summed per
    key over workers and rounds, pulls return (n, k) arrays, channels do not mix."""
    from parameter_server_b200.parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig, heap_layout
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.parameter.kv import DeviceKVVector
    pc = PlaneConfig(table_capacity=1 << 12, inbox_cap=1 << 10, ring=4, pull_cap=1 << 10, width=k, channels=2, quant=quant)
    fabs = Fabric.emulated(S, heap_layout(pc, S).total())
    kvs = [DeviceKVVector(DataPlane(f, pc, OptimizerConfig(algo="sum")), 1 << 10) for f in fabs]
    rng = np.random.default_rng(S * 100 + k)
    universe = np.unique(rng.integers(0, np.iinfo(np.uint64).max, 600, dtype=np.uint64))
    state = [dict(), dict()]
    for rnd in range(3):
        chl = rnd % 2
        per = []
        for r in range(S):
            keys = np.sort(rng.choice(universe, 150, replace=False))
            vals = rng.normal(size=(len(keys), k)).astype(np.float32)
            per.append((keys, vals))
            for kk, vv in zip(keys.tolist(), vals):
                state[chl][kk] = state[chl].get(kk, np.zeros(k, np.float32)) + vv
        for r in range(S):               # emulated ranks: every worker's push first, then every owner's apply
            kv = kvs[r]
            b = kv._buffer(kv._as_keys(per[r][0], kv.dev))
            b.grad[:per[r][1].size].copy_(torch.from_numpy(per[r][1]).flatten())
            kv.plane.push(b, rnd, with_gradient=False)
        for r in range(S):
            kvs[r].plane.apply(rnd, channel=chl)
    tol = dict(rtol=1e-4, atol=1e-5) if quant == "none" else dict(rtol=0.05, atol=0.05)
    for chl in range(2):
        ask = np.sort(rng.choice(universe, 200, replace=False))
        stamps = []
        for phase in (1, 2, 4):          # the three roles of the exchange pull as separate launches
            for r in range(S):
                kv = kvs[r]
                b = kv._buffer(kv._as_keys(ask if r == 0 else np.zeros(0, np.uint64), kv.dev))
                kv.plane.pull_exchange(b, chl, need_applied=3, with_margins=False, channel=chl, phases=phase,
                                       wait_iters=1 << 12)
        torch.cuda.synchronize()
        got = kvs[0].plane.response_weights(chl, len(ask)).cpu().numpy()
        exp = np.stack([state[chl].get(kk, np.zeros(k, np.float32)) for kk in ask.tolist()])
        assert got.shape == (len(ask), k)
        assert np.allclose(got, exp, **tol), float(np.abs(got - exp).max())
    for kv in kvs:
        kv.plane.check_status()


def test_buffered_kv_vector_aggregation_idiom(cuda_lib):
    """buffer_value=True: a push round is kept per source for the owner to look at; the owner merges it
    explicitly; a later pull sees the merged sum (test/kv_vector_buffer_ps.cc:10-59)."""
    from parameter_server_b200.parameter.kv import DeviceKVVector
    kv = DeviceKVVector.create(table_capacity=1 << 12, max_keys=1 << 10, k=2, buffer_value=True)
    keys = np.array([5, 9, 1 << 50], dtype=np.uint64)
    vals = np.array([[1, 2], [3, 4], [5, 6]], dtype=np.float32)
    t0 = kv.push(keys, vals)
    t1 = kv.pull(keys)
    kv.wait(t1)
    assert float(kv.result(t1).abs().sum()) == 0.0            # nothing merged yet
    (bk, bv), = kv.buffer(t0)
    assert np.array_equal(bk, keys) and np.array_equal(bv.cpu().numpy(), vals)
    kv.apply_buffer(t0)
    kv.apply_buffer(t0)                                      # merging is the owner's decision: here twice
    t2 = kv.pull(keys)
    kv.wait(t2)
    assert np.array_equal(kv.result(t2).cpu().numpy(), 2 * vals)
