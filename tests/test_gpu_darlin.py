"""Darlin device kernels against the NumPy restatement, single rank and emulated shards."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _data(rng, rows, z, n_feat, real):
    from parameter_server_b200.utils.oracle import hash_id_to_key
    ids = np.minimum((rng.pareto(1.1, rows * z) * 2).astype(np.int64), n_feat - 1)
    keys = hash_id_to_key(ids, 5)
    w_star = np.where(rng.random(n_feat) < 0.1, rng.normal(0, 2, n_feat), 0)
    vals = (np.abs(rng.normal(0, 1, rows * z)) + 0.1).astype(np.float32) if real else None
    x = vals if real else 1.0
    margin = (w_star[ids] * x).reshape(rows, z).sum(1)
    y = np.where(margin + rng.logistic(size=rows) >= 0, 1.0, -1.0).astype(np.float32)
    return keys, y, vals


@pytest.mark.parametrize("S,real", [(1, False), (1, True), (2, False), (4, True)])
def test_darlin_matches_oracle(cuda_lib, S, real):
    from parameter_server_b200.models.darlin import DarlinConfig, DarlinRank, darlin_heap_bytes, run_darlin
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.utils import oracle
    rng = np.random.default_rng(10 + S)
    rows, z, n_feat = 600, 10, 300
    cfg = DarlinConfig(lambda_l1=1.0, eta=0.9, block_cols=64, max_pass=4, epsilon=0.0, random_block_order=True, kkt_ratio=10.0)
    fabs = Fabric.emulated(S, darlin_heap_bytes(cfg, S))
    parts = [_data(rng, rows, z, n_feat, real) for _ in range(S)]
    gk = np.unique(np.concatenate([p[0] for p in parts]))
    gkt = torch.from_numpy(gk.view(np.int64)).cuda()
    ranks = []
    for f, (keys, y, vals) in zip(fabs, parts):
        ranks.append(DarlinRank(f, cfg, torch.from_numpy(keys.view(np.int64)).cuda(), torch.from_numpy(y).cuda(), fixed_z=z,
                                vals=None if vals is None else torch.from_numpy(vals).cuda(), global_keys=gkt))
    hist = run_darlin(ranks)
    torch.cuda.synchronize()
    blocks = ranks[0].blocks
    orders = []
    for it in range(cfg.max_pass):
        o = list(range(len(blocks))); np.random.default_rng(1000 + it).shuffle(o)
        orders.append([blocks[i] for i in o])
    row_ptr = np.arange(rows + 1) * z
    w_ref, h_ref = oracle.darlin_oracle([(k, row_ptr, y, v) for k, y, v in parts], gk, cfg.lambda_l1, cfg.eta,
                                        cfg.delta_init, cfg.delta_max, orders, cfg.max_pass, cfg.kkt_ratio)
    assert np.allclose([h["objective"] for h in hist], h_ref, rtol=2e-4)
    got = np.zeros(len(gk), np.float32)
    for r in ranks:
        k, w = r.my_model()
        got[np.searchsorted(gk, k)] = w
    assert np.allclose(got, np.where(np.isnan(w_ref), 0, w_ref), rtol=2e-3, atol=2e-4)
    assert min(h["objective"] for h in hist) < rows * S * np.log(2)
    assert 0 < hist[-1]["nnz_w"] < len(gk)


@pytest.mark.parametrize("S,real", [(1, False), (2, True)])
def test_darlin_warm_start_matches_oracle(cuda_lib, S, real):
    """set_initial_weights (the reference's init_w): margins start at X w0, and the passes that follow match
    the NumPy restatement started from the same weights."""
    from parameter_server_b200.models.darlin import DarlinConfig, DarlinRank, darlin_heap_bytes, run_darlin
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.utils import oracle
    rng = np.random.default_rng(40 + S)
    rows, z, n_feat = 500, 8, 250
    cfg = DarlinConfig(lambda_l1=1.0, eta=0.3, block_cols=64, max_pass=3, epsilon=0.0, random_block_order=True, kkt_ratio=10.0)
    fabs = Fabric.emulated(S, darlin_heap_bytes(cfg, S))
    parts = [_data(rng, rows, z, n_feat, real) for _ in range(S)]
    gk = np.unique(np.concatenate([p[0] for p in parts]))
    gkt = torch.from_numpy(gk.view(np.int64)).cuda()
    w0 = (np.full(len(gk), 0.05, np.float32) if S == 1 else
          np.random.RandomState(7).normal(0, 0.1, len(gk)).astype(np.float32))
    ranks = []
    for f, (keys, y, vals) in zip(fabs, parts):
        r = DarlinRank(f, cfg, torch.from_numpy(keys.view(np.int64)).cuda(), torch.from_numpy(y).cuda(), fixed_z=z,
                       vals=None if vals is None else torch.from_numpy(vals).cuda(), global_keys=gkt)
        r.set_initial_weights(torch.from_numpy(w0))
        x = np.ones(rows * z, np.float32) if vals is None else vals
        want = (w0[np.searchsorted(gk, keys)] * x).reshape(rows, z).sum(1)
        assert np.allclose(r.margin.cpu().numpy(), want, rtol=1e-4, atol=1e-5)
        ranks.append(r)
    hist = run_darlin(ranks)
    torch.cuda.synchronize()
    blocks = ranks[0].blocks
    orders = []
    for it in range(cfg.max_pass):
        o = list(range(len(blocks))); np.random.default_rng(1000 + it).shuffle(o)
        orders.append([blocks[i] for i in o])
    row_ptr = np.arange(rows + 1) * z
    w_ref, h_ref = oracle.darlin_oracle([(k, row_ptr, y, v) for k, y, v in parts], gk, cfg.lambda_l1, cfg.eta,
                                        cfg.delta_init, cfg.delta_max, orders, cfg.max_pass, cfg.kkt_ratio, w0=w0)
    assert np.allclose([h["objective"] for h in hist], h_ref, rtol=2e-4)
    got = np.zeros(len(gk), np.float32)
    for r in ranks:
        k, w = r.my_model()
        got[np.searchsorted(gk, k)] = w
    assert np.allclose(got, np.where(np.isnan(w_ref), 0, w_ref), rtol=2e-3, atol=2e-4)


def test_darlin_bounded_delay_single_rank_converges(cuda_lib):
    from parameter_server_b200.models.darlin import DarlinConfig, DarlinRank, darlin_heap_bytes, run_darlin
    from parameter_server_b200.parallel.fabric import Fabric
    rng = np.random.default_rng(3)
    keys, y, _ = _data(rng, 4000, 12, 2000, False)
    objs = {}
    for tau in (0, 2):
        cfg = DarlinConfig(lambda_l1=1.0, eta=0.3, block_cols=8, max_pass=8, epsilon=1e-5, tau=tau)
        fab = Fabric.single(darlin_heap_bytes(cfg, 1))
        r = DarlinRank(fab, cfg, torch.from_numpy(keys.view(np.int64)).cuda(), torch.from_numpy(y).cuda(), fixed_z=12)
        hist = run_darlin([r])
        objs[tau] = hist[-1]["objective"]
        assert hist[-1]["objective"] < 0.95 * 4000 * np.log(2)       # well below the zero model
        assert hist[-1]["objective"] <= hist[0]["objective"]
    assert abs(objs[0] - objs[2]) / objs[0] < 0.05


def test_device_preprocessing_tail_filter_groups_and_blocks(cuda_lib):
    """Column space, tail filter and block division on the device against NumPy: two feature groups,
    keys below the frequency threshold dropped, columns group-major with keys ascending inside a
    group, blocks per group from nnz per row, prior group first."""
    from parameter_server_b200.models.darlin_prep import build_columns, plan_blocks
    rng = np.random.default_rng(0)
    rows = 500
    groups = []
    for gid, (n_feat, z) in enumerate([(40, 3), (3000, 6)]):
        lens = rng.integers(1, 2 * z, rows)
        off = np.concatenate([[0], np.cumsum(lens)])
        ids = np.minimum((rng.pareto(1.0, off[-1]) * 3).astype(np.int64), n_feat - 1)
        keys = (ids.astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15)) ^ np.uint64(gid << 60)
        groups.append(dict(id=gid, offset=off, index=keys, value=np.zeros(0, np.float32), binary=True))
    col, row_ptr, vals, space = build_columns(groups, rows, "cuda", tail_freq=4, countmin_cells=1 << 20, countmin_k=2)
    assert vals is None and len(space.groups) == 2
    base = 0
    exp_rows = [[] for _ in range(rows)]
    for g in groups:
        u, cnt = np.unique(g["index"], return_counts=True)
        kept = u[cnt >= 4]                                   # the sketch is large: estimates are exact here
        gid, c0, c1 = space.groups[g["id"]]
        assert (c0, c1) == (base, base + len(kept))
        assert np.array_equal(space.col_key[c0:c1].cpu().numpy().view(np.uint64), kept)
        for r in range(rows):
            ks = g["index"][g["offset"][r]:g["offset"][r + 1]]
            exp_rows[r] += [base + int(np.searchsorted(kept, k)) for k in ks if k in set(kept.tolist())]
        base += len(kept)
    rp = row_ptr.cpu().numpy()
    c = col.cpu().numpy()
    for r in range(0, rows, 7):
        assert sorted(c[rp[r]:rp[r + 1]].tolist()) == sorted(exp_rows[r]), r
    assert space.dropped_nnz == sum(len(g["index"]) for g in groups) - len(c) > 0
    plan = plan_blocks(space, feature_block_ratio=2.0, max_block_cols=64, prior_groups=[0], prior_iters=3)
    assert all(b1 - b0 <= 64 for b0, b1 in plan.blocks) and plan.block_cols <= 64
    assert [b for b, g in zip(plan.blocks, plan.group_of) if g == 0][0][0] == 0
    n0 = sum(1 for g in plan.group_of if g == 0)
    assert plan.prior == list(range(n0)) * 3
    # every column is in exactly one block, blocks never straddle a group
    covered = np.zeros(space.n_cols, int)
    for (b0, b1), g in zip(plan.blocks, plan.group_of):
        covered[b0:b1] += 1
        gid, c0, c1 = space.groups[g]
        assert c0 <= b0 and b1 <= c1
    assert (covered == 1).all()
