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
    assert sum(big) == 100_003 and max(big) - min(big) <= 7     # boundaries are multiples of four elements


def test_kvlayer_ring_bounds_a_fast_worker(cuda_lib):
    """Two emulated ranks, ring of two slots: worker 0 may push rounds 0 and 1 before anybody applies;
    its push of round 2 would overwrite the slot of round 0, so it waits for the owner's applied
    counter and, with a short budget and nobody applying, reports a timeout instead of overwriting."""
    from parameter_server_b200.ops._lib import PsbCudaError
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.parameter.kv_layer import DeviceKVLayer
    layers = {0: 4096}
    fabs = Fabric.emulated(2, DeviceKVLayer.heap_bytes(layers, 2))
    kv = [DeviceKVLayer(f, layers, updater="add", ring=2) for f in fabs]
    g = [torch.full((4096,), float(r + 1), device="cuda") for r in range(2)]
    for rnd in range(2):
        for r in range(2):
            kv[r].push(0, g[r] * (rnd + 1))
    torch.cuda.synchronize()
    kv[0].check_status(); kv[1].check_status()
    kv[0].push(0, g[0] * 100, wait_iters=2000)      # round 2: slot of round 0 is not applied yet
    torch.cuda.synchronize()
    with pytest.raises(PsbCudaError):
        kv[0].check_status()
    # the owners now apply rounds 0 and 1: each sums exactly that round's data
    for rnd in range(2):
        for r in range(2):
            kv[r].apply(0)
    out = torch.zeros(4096, device="cuda")
    kv[1].pull(0, out, wait_for_round=2)
    torch.cuda.synchronize()
    kv[1].check_status()
    # the push that timed out touched nothing: rounds 0 and 1 of both workers sum to (1 + 2) * (1 + 2)
    assert torch.equal(out, torch.full_like(out, 9.0))
