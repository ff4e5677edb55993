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
