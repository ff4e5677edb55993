"""Device filters against their host (C++) counterparts."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_key_signature_matches_host_crc_and_detects_repeats(cuda_lib):
    from parameter_server_b200.ops._lib import check, ptr, stream_ptr
    from parameter_server_b200.system import core
    dev = torch.device("cuda")
    rng = np.random.default_rng(0)
    state = torch.zeros(4, dtype=torch.int32, device=dev)
    scratch = torch.zeros(4, dtype=torch.int32, device=dev)
    hit = torch.zeros(1, dtype=torch.int32, device=dev)
    sig = torch.zeros(4, dtype=torch.int32, device=dev)
    lists = [np.sort(rng.integers(0, 1 << 62, n, dtype=np.uint64)) for n in (10, 5000, 5000)]
    lists.insert(2, lists[1].copy())                       # a repeat
    tail_changed = lists[1].copy(); tail_changed[-1] += 1  # differs only beyond the first 2 KiB
    lists.append(tail_changed)
    hits = []
    for k in lists:
        kt = torch.from_numpy(k.view(np.int64)).to(dev)
        n = torch.tensor([len(k)], dtype=torch.int32, device=dev)
        check(cuda_lib.psb_key_signature(ptr(kt), ptr(n), len(k), ptr(scratch), ptr(state), ptr(hit), ptr(sig), stream_ptr()))
        hits.append(int(hit.item()))
        crc = int(sig[0].item()) & 0xFFFFFFFF
        assert crc == core.crc32c(k.tobytes()[:2048])
    assert hits == [0, 0, 1, 0, 0]


@pytest.mark.parametrize("nbytes", [1, 2, 3])
def test_fixing_float_codec_error_bound_and_host_decode(cuda_lib, nbytes):
    from parameter_server_b200.ops.filters import fixing_float_decode, fixing_float_encode
    x = torch.randn(10001, device="cuda") * 3
    code, lo, hi = fixing_float_encode(x, nbytes, seed=5)
    y = fixing_float_decode(code, nbytes, lo, hi)
    step = (hi - lo) / (2 ** (8 * nbytes) - 2)
    assert float((x - y).abs().max()) <= step * 1.001 + 1e-6
    # the host decoder of the reference codec reads the same bytes
    ratio = float(2 ** (8 * nbytes) - 2)
    c = code.cpu().numpy().reshape(-1, nbytes).astype(np.uint64)
    r = sum(c[:, j] << np.uint64(8 * j) for j in range(nbytes)).astype(np.float64)
    host = (r / ratio * (hi - lo) + lo).astype(np.float32)
    assert np.allclose(host, y.cpu().numpy(), atol=1e-6)
    with pytest.raises(Exception):
        fixing_float_encode(x, 9)


def test_countmin_matches_host_sketch(cuda_lib):
    from parameter_server_b200.ops.filters import CountMin
    from parameter_server_b200.system import core
    rng = np.random.default_rng(1)
    keys = np.unique(rng.integers(0, 1 << 60, 5000, dtype=np.uint64))
    counts = rng.integers(1, 200, len(keys)).astype(np.uint8)
    host = core.CountMin(); host.resize(4096, 2, 255)
    host.insert_many(keys, counts)
    dev = CountMin(4096, 2)
    dev.insert(torch.from_numpy(keys.view(np.int64)).cuda(), torch.from_numpy(counts).cuda())
    assert np.array_equal(dev.bytes().cpu().numpy(), host.data())
    q = dev.query(torch.from_numpy(keys.view(np.int64)).cuda()).cpu().numpy()
    assert np.array_equal(q, host.query_many(keys))
    assert (q >= counts).all()


@pytest.mark.parametrize("k,op", [(1, 0), (2, 1), (4, 2)])
def test_ordered_match_matches_host(cuda_lib, k, op):
    from parameter_server_b200.ops.filters import ordered_match
    from parameter_server_b200.system import core
    rng = np.random.default_rng(k)
    universe = np.unique(rng.integers(0, 1 << 40, 4000, dtype=np.uint64))
    src = np.sort(rng.choice(universe, 1500, replace=False)); dst = np.sort(rng.choice(universe, 2500, replace=False))
    sv = rng.random(len(src) * k, dtype=np.float32); dv = rng.random(len(dst) * k, dtype=np.float32)
    n_host, exp = core.ordered_match(src, sv, dst, dv, k, op, 2)
    d = torch.from_numpy(dv.copy()).cuda()
    n = ordered_match(torch.from_numpy(src.view(np.int64)).cuda(), torch.from_numpy(sv).cuda(),
                      torch.from_numpy(dst.view(np.int64)).cuda(), d, k, op)
    assert n == n_host == len(np.intersect1d(src, dst))
    assert np.allclose(d.cpu().numpy(), exp)


def test_key_cache_training_equals_uncached(cuda_lib):
    """Repeating the same minibatch with the key cache on (values-only pushes,
    probe-free pulls) gives the same model as with it off."""
    from parameter_server_b200.models.sparse_lr import SparseLRConfig, SparseLRWorker
    from parameter_server_b200.parallel.dataplane import DataPlane, OptimizerConfig, PlaneConfig, heap_layout
    from parameter_server_b200.parallel.fabric import Fabric
    rng = np.random.default_rng(3)
    rows, z = 256, 16
    ids = torch.from_numpy(rng.integers(0, 3000, rows * z).astype(np.int32)).cuda()
    y = torch.from_numpy(np.where(rng.random(rows) < 0.5, 1.0, -1.0).astype(np.float32)).cuda()
    ids2 = torch.from_numpy(rng.integers(0, 3000, rows * z).astype(np.int32)).cuda()
    outs = []
    for cache in (False, True):
        planes = []
        pc = PlaneConfig(table_capacity=1 << 14, inbox_cap=rows * z, ring=2, key_cache=cache, ordered_slots=True)
        fabs = Fabric.emulated(2, heap_layout(pc, 2).total())
        planes = [DataPlane(f, pc, OptimizerConfig(algo="ftrl", l1=0.01)) for f in fabs]
        ws = [SparseLRWorker(p, SparseLRConfig(max_rows=rows, max_nnz=rows * z, hash_seed=2, pipeline=1)) for p in planes]
        hits = []
        for step, batch in enumerate([ids, ids, ids, ids2, ids2, ids]):
            bs = []
            for w in ws:
                b = w.prepare(batch, y, fixed_z=z)
                if cache:
                    w.plane.key_signature(b)
                w.plane.pull_margin(b, need_applied=step)
                bs.append(b)
            for w, b in zip(ws, bs):
                w.plane.push(b, step)
            for w in ws:
                w.plane.apply(step)
                w.step_no += 1
            hits.append(int(bs[0].key_hit.item()))
        torch.cuda.synchronize()
        for p in planes:
            p.check_status()
        if cache:
            assert hits == [0, 1, 1, 0, 1, 0]
        outs.append([p.dump_nonzero() for p in planes])
    for (k0, w0), (k1, w1) in zip(*outs):
        assert np.array_equal(k0.numpy(), k1.numpy())
        assert np.allclose(w0.numpy(), w1.numpy(), rtol=1e-5, atol=1e-7)
