"""Device KVLayer: placement rule, push (sum over workers + updater) and pull."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S,updater", [(1, "add"), (3, "add"), (4, "sgd")])
def test_kvlayer_push_pull(cuda_lib, S, updater):
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.parameter.kv_layer import DeviceKVLayer
    layers = {0: 10, 1: 64, 2: 100_003, 7: 999}
    fabs = Fabric.emulated(S, DeviceKVLayer.heap_bytes(layers, S))
    kv = [DeviceKVLayer(f, layers, partition_thr=1000, updater=updater, lr=0.5) for f in fabs]
    rng = np.random.default_rng(S)
    state = {lid: np.zeros(n, np.float32) for lid, n in layers.items()}
    for rnd in range(2):
        for lid, n in layers.items():
            grads = [rng.normal(size=n).astype(np.float32) for _ in range(S)]
            for r in range(S):
                kv[r].push(lid, torch.from_numpy(grads[r]).cuda())
            for r in range(S):
                kv[r].apply(lid)
            total = np.sum(grads, axis=0)
            state[lid] = state[lid] + total if updater == "add" else state[lid] - 0.5 * total
    for lid, n in layers.items():
        for r in (0, S - 1):
            out = torch.zeros(n, device="cuda")
            kv[r].pull(lid, out, wait_for_round=2)
            torch.cuda.synchronize()
            kv[r].check_status()
            assert np.allclose(out.cpu().numpy(), state[lid], rtol=1e-5, atol=1e-5), lid
    # placement: a small layer lives whole on (id * 991) % S, a large one is split evenly
    sizes = [len(k.segment(7)) for k in kv]
    assert sorted(sizes)[-1] == 999 and sum(sizes) == 999 and sizes[(7 * 991) % S] == 999
    big = [len(k.segment(2)) for k in kv]
    assert sum(big) == 100_003 and max(big) - min(big) <= 1
