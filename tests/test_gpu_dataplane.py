"""Fused pull / push / apply kernels against the NumPy oracle, on one GPU and on
several emulated shards of one GPU (kernels of different virtual ranks run one
after another on one stream)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(S, opt, cap=1 << 14, inbox=1 << 13, ring=3, quant="none", ordered=False, pull_cap=0):
    from parameter_server_b200.parallel.dataplane import DataPlane, PlaneConfig, heap_layout
    from parameter_server_b200.parallel.fabric import Fabric
    pc = PlaneConfig(table_capacity=cap, inbox_cap=inbox, ring=ring, quant=quant, ordered_slots=ordered,
                     pull_cap=pull_cap)
    fabs = Fabric.emulated(S, heap_layout(pc, S).total())
    return [DataPlane(f, pc, opt) for f in fabs]


def _batch(rng, rows, z, n_feat, seed=1):
    from parameter_server_b200.utils.oracle import hash_id_to_key
    ids = np.minimum((rng.pareto(1.05, rows * z) * 2).astype(np.int64), n_feat - 1).astype(np.int32)
    y = np.where(rng.random(rows) < 0.5, 1.0, -1.0).astype(np.float32)
    return ids, y, hash_id_to_key(ids, seed)


@pytest.mark.parametrize("ordered", [False, True])
@pytest.mark.parametrize("algo", ["ftrl", "adagrad", "sgd"])
def test_single_shard_training_matches_oracle(cuda_lib, algo, ordered):
    from parameter_server_b200.models.sparse_lr import SparseLRConfig, SparseLRWorker
    from parameter_server_b200.parallel.dataplane import OptimizerConfig
    from parameter_server_b200.utils import oracle
    opt = OptimizerConfig(algo=algo, alpha=0.1, beta=1.0, l1=0.01, l2=0.1)
    plane = _mk(1, opt, ordered=ordered)[0]
    rows, z = 256, 24
    w = SparseLRWorker(plane, SparseLRConfig(max_rows=rows, max_nnz=rows * z, tau=0, hash_seed=1, pipeline=1))
    ot = oracle.OracleTable(opt)
    rng = np.random.default_rng(0)
    row_ptr = np.arange(rows + 1) * z
    tot = 0.0
    for step in range(6):
        ids, y, keys = _batch(rng, rows, z, 3000)
        b = w.step(torch.from_numpy(ids).cuda(), torch.from_numpy(y).cuda(), fixed_z=z)
        loss, margin, u, grad = oracle.sparse_lr_step(ot, keys, row_ptr, y)
        tot += loss
        torch.cuda.synchronize()
        plane.check_status()
        assert np.allclose(b.margin[:rows].cpu().numpy(), margin, rtol=1e-4, atol=1e-5), step
        U = int(b.n_unique.item())
        assert np.allclose(b.grad[:U].cpu().numpy(), grad, rtol=1e-4, atol=1e-5)
    prog = w.read_progress()
    assert prog["n_examples"] == 6 * rows
    assert abs(prog["loss_sum"] - tot) < 1e-3 * tot
    k, wv = plane.dump_nonzero()
    ok, ow = ot.nonzero()
    assert np.array_equal(k.numpy(), ok)
    assert np.allclose(wv.numpy(), ow, rtol=2e-4, atol=1e-6)


@pytest.mark.parametrize("S", [2, 4])
@pytest.mark.parametrize("quant", ["none", "int8", "fp16"])
def test_emulated_shards_aggregate_pushes(cuda_lib, S, quant):
    """S workers push the same round; every owner sums duplicate keys across
    sources and runs FTRL once on the sum."""
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.parallel.dataplane import OptimizerConfig
    from parameter_server_b200.utils import oracle
    opt = OptimizerConfig(algo="ftrl", alpha=0.1, beta=1.0, l1=0.001, l2=0.1)
    planes = _mk(S, opt, quant=quant, ordered=(S == 4))
    rows, z = 128, 16
    rng = np.random.default_rng(S)
    ot = oracle.OracleTable(opt)
    bufs = [LocalBatch(rows, rows * z, S, "cuda") for _ in range(S)]
    row_ptr = np.arange(rows + 1) * z
    for t in range(4):
        data = [_batch(rng, rows, z, 2000) for _ in range(S)]
        # oracle: pull (same weights for all), per-worker gradients, summed per key, one step
        gsum = {}
        for ids, y, keys in data:
            u, col, _ = oracle.localize(keys)
            wv = ot.pull(u)
            margin = np.add.reduceat(wv[col].astype(np.float64), row_ptr[:-1]).astype(np.float32)
            _, gc = oracle.logit_loss_and_gcoef(y, margin)
            g = np.zeros(len(u)); np.add.at(g, col, gc[np.repeat(np.arange(rows), z)])
            g = g.astype(np.float32)
            if quant != "none":
                # quantise per (owner, source) inbox, groups of 32 records
                bh = planes[0].bounds_host
                offs = [int(np.searchsorted(u, np.uint64(x))) for x in bh[:-1]] + [len(u)]
                for s in range(S):
                    g[offs[s]:offs[s + 1]] = oracle.block_quantize(g[offs[s]:offs[s + 1]], quant)
            for k, v in zip(u.tolist(), g.tolist()):
                gsum[k] = gsum.get(k, 0.0) + v
        ks = np.array(sorted(gsum), dtype=np.uint64)
        ot.push(ks, np.array([gsum[k] for k in ks.tolist()], dtype=np.float32))
        for r in range(S):
            ids, y, _ = data[r]
            bufs[r].localize(torch.from_numpy(ids).cuda(), torch.from_numpy(y).cuda(), planes[r].bounds,
                             fixed_z=z, hash_seed=1)
            planes[r].pull_margin(bufs[r], need_applied=t)
        for r in range(S):
            planes[r].push(bufs[r], t)
        for r in range(S):
            planes[r].apply(t)
        torch.cuda.synchronize()
        for p in planes:
            p.check_status()
    got = {}
    for p in planes:
        k, wv = p.dump_nonzero()
        lo, hi = p.bounds_host[p.rank], p.bounds_host[p.rank + 1]
        assert all(lo <= int(x) < hi for x in k.numpy().tolist())
        got.update(zip(k.numpy().tolist(), wv.numpy().tolist()))
    ok, ow = ot.nonzero()
    # quantisation is emulated exactly in the oracle; what remains is summation
    # order, plus rare rounding ties in v/scale
    tol = dict(none=(2e-4, 1e-6), int8=(2e-3, 1e-4), fp16=(2e-3, 1e-4))[quant]
    exp = dict(zip(ok.tolist(), ow.tolist()))
    if quant == "none":
        assert sorted(got) == ok.tolist()
    common = [k for k in exp if k in got]
    assert len(common) > 0.98 * len(exp)
    a = np.array([got[k] for k in common]); b_ = np.array([exp[k] for k in common])
    close = np.isclose(a, b_, rtol=tol[0], atol=tol[1])
    assert close.mean() > (0.999 if quant == "none" else 0.98), (close.mean(), np.abs(a - b_).max())


def test_dead_source_is_skipped_and_wait_times_out_cleanly(cuda_lib):
    """A source that never pushes: with alive=False the apply completes; with
    alive=True the bounded wait runs out and reports status 3 (no hang)."""
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.ops._lib import PsbCudaError
    from parameter_server_b200.parallel.dataplane import OptimizerConfig
    opt = OptimizerConfig(algo="sum")
    planes = _mk(2, opt)
    b = LocalBatch(8, 64, 2, "cuda")
    keys = np.array([5, 1 << 63, (1 << 63) + 9], dtype=np.uint64)
    b.set_keys(torch.from_numpy(keys.view(np.int64)).cuda(), planes[0].bounds)
    b.grad[:3] = torch.tensor([1.0, 2.0, 3.0]).cuda()
    planes[0].push(b, 0, with_gradient=False)       # rank 1 never pushes
    planes[1].set_alive(1, False)
    planes[1].apply(0)
    torch.cuda.synchronize()
    planes[1].check_status()
    k, w = planes[1].dump_nonzero()
    assert k.numpy().tolist() == [1 << 63, (1 << 63) + 9] and w.tolist() == [2.0, 3.0]
    planes[0].apply(0, wait_iters=2000)              # waits for rank 1's flag: bounded
    torch.cuda.synchronize()
    with pytest.raises(PsbCudaError, match="timed out"):
        planes[0].check_status()
    # the context is still usable
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_pipelined_submit_matches_synchronous(cuda_lib):
    from parameter_server_b200.models.sparse_lr import SparseLRConfig, SparseLRWorker
    from parameter_server_b200.parallel.dataplane import OptimizerConfig
    opt = OptimizerConfig(algo="ftrl", l1=0.01)
    rows, z = 512, 20
    rng = np.random.default_rng(2)
    batches = [_batch(rng, rows, z, 5000) for _ in range(5)]
    outs = []
    for mode in ("sync", "pipe"):
        plane = _mk(1, opt, ring=2)[0]
        w = SparseLRWorker(plane, SparseLRConfig(max_rows=rows, max_nnz=rows * z, tau=0, hash_seed=1, pipeline=2))
        for ids, y, _ in batches:
            if mode == "sync":
                w.step(torch.from_numpy(ids).cuda(), torch.from_numpy(y).cuda(), fixed_z=z)
            else:
                w.submit(torch.from_numpy(ids).pin_memory(), torch.from_numpy(y).pin_memory(), fixed_z=z)
        w.wait()
        torch.cuda.synchronize()
        plane.check_status()
        outs.append(plane.dump_nonzero())
    assert np.array_equal(outs[0][0].numpy(), outs[1][0].numpy())
    assert np.allclose(outs[0][1].numpy(), outs[1][1].numpy(), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("S,hashed", [(1, True), (3, True), (8, True), (2, False)])
def test_pull_exchange_equals_one_sided_path(cuda_lib, S, hashed):
    """Two-sided pull (keys to owners, weights back, slots reused by a values-only
    push) gives the same margins and the same model as the one-sided path. The
    three phases run as separate launches here because the emulated ranks share
    one GPU and one stream. With several sources the exchange path merges the
    sources' records per key-range part in shared memory, the one-sided path
    accumulates in the table and lets one record per key lead: both must agree,
    with eight sources too. ``hashed=False``: small consecutive keys, which all
    fall into the first part of the first owner, more than the merge table takes,
    so that part goes through the accumulate-then-lead protocol inside the
    exchange path."""
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.parallel.dataplane import OptimizerConfig
    opt = OptimizerConfig(algo="ftrl", alpha=0.1, beta=1.0, l1=0.01, l2=0.1)
    rows, z = 128, 16
    rng = np.random.default_rng(40 + S)
    rounds = [[_batch(rng, rows, z, 2000) for _ in range(S)] for _ in range(4)]
    results = []
    for mode in ("one_sided", "exchange"):
        planes = _mk(S, opt, pull_cap=rows * z if mode == "exchange" else 0, ordered=hashed, inbox=rows * z)
        bufs = [LocalBatch(rows, rows * z, S, "cuda") for _ in range(S)]
        margins = []
        for t, data in enumerate(rounds):
            for r in range(S):
                ids, y, _ = data[r]
                if hashed:
                    bufs[r].localize(torch.from_numpy(ids).cuda(), torch.from_numpy(y).cuda(), planes[r].bounds, fixed_z=z, hash_seed=1)
                else:
                    bufs[r].localize(torch.from_numpy(ids.astype(np.int64) + 1).cuda(), torch.from_numpy(y).cuda(),
                                     planes[r].bounds, fixed_z=z, hash_seed=None)
            if mode == "one_sided":
                for r in range(S):
                    planes[r].pull_margin(bufs[r], need_applied=t)
                for r in range(S):
                    planes[r].push(bufs[r], t)
            else:
                for ph in (1, 2, 4):
                    for r in range(S):
                        planes[r].pull_exchange(bufs[r], t, need_applied=t, phases=ph)
                for r in range(S):
                    planes[r].push(bufs[r], t, send_keys=False)
            for r in range(S):
                planes[r].apply(t)
            torch.cuda.synchronize()
            for p in planes:
                p.check_status()
            margins.append(torch.stack([b.margin[:rows].clone() for b in bufs]).cpu())
        results.append((margins, [p.dump_nonzero() for p in planes]))
    for a, b in zip(results[0][0], results[1][0]):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
    for (k0, w0), (k1, w1) in zip(results[0][1], results[1][1]):
        assert np.array_equal(k0.numpy(), k1.numpy())
        assert np.allclose(w0.numpy(), w1.numpy(), rtol=1e-4, atol=1e-6)


def test_checkpoint_resume_equals_uninterrupted_run(cuda_lib, tmp_path):
    """Train 3 steps, checkpoint (weights and FTRL z/n), load into a fresh plane with a
    different number of shards, train 3 more: same model as 6 uninterrupted steps."""
    from parameter_server_b200.models.sparse_lr import SparseLRConfig, SparseLRWorker
    from parameter_server_b200.parallel.dataplane import OptimizerConfig
    from parameter_server_b200.utils import checkpoint as ck
    opt = OptimizerConfig(algo="ftrl", alpha=0.1, beta=1.0, l1=0.01, l2=0.1)
    rows, z = 128, 16
    rng = np.random.default_rng(4)
    data = [_batch(rng, rows, z, 4000)[:2] for _ in range(6)]

    def worker(plane):
        return SparseLRWorker(plane, SparseLRConfig(max_rows=rows, max_nnz=rows * z, tau=0, hash_seed=1, pipeline=1))

    def run(w, batches):
        for ids, y in batches:
            w.step(torch.from_numpy(ids).cuda(), torch.from_numpy(y).cuda(), fixed_z=z)
        torch.cuda.synchronize()

    ref = worker(_mk(1, opt)[0])
    run(ref, data)
    k_ref, w_ref = ref.plane.dump_nonzero()

    a = worker(_mk(1, opt)[0])
    run(a, data[:3])
    prefix = str(tmp_path / "ckpt")
    ck.save_plane(a.plane, prefix, meta={"step": 3})
    b = worker(_mk(1, opt, ordered=True)[0])
    assert ck.load_plane(b.plane, prefix)["step"] == 3
    run(b, data[3:])
    k_b, w_b = b.plane.dump_nonzero()
    assert torch.equal(k_ref, k_b)
    assert torch.allclose(w_ref, w_b, rtol=1e-6, atol=1e-7)
