"""Wide-value path: tcgen05 pull+GEMM, row sums, push and AdaGrad apply against PyTorch fp32."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(S, N, rows=300, z=12, n_feat=2500, seed=0, pull_cap=0):
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.parallel.fabric import Fabric
    from parameter_server_b200.parallel.wide import WideConfig, WidePlane, wide_layout
    from parameter_server_b200.utils.oracle import hash_id_to_key
    rng = np.random.default_rng(seed)
    cfg = WideConfig(table_capacity=1 << 13, inbox_cap=rows * z, ring=2, alpha=0.1, beta=1.0, pull_cap=pull_cap)
    fabs = Fabric.emulated(S, wide_layout(cfg, S).total())
    planes = [WidePlane(f, cfg) for f in fabs]
    all_ids = np.arange(n_feat)
    all_keys = hash_id_to_key(all_ids, 11)
    table = (torch.randn(n_feat, 64) * 0.5).to(torch.bfloat16)
    known = rng.random(n_feat) < 0.8                  # 20 % of the keys are not in the table yet
    for p in planes:
        lo, hi = p.bounds_host[p.rank], p.bounds_host[p.rank + 1]
        sel = known & (all_keys >= np.uint64(lo)) & (all_keys < np.uint64(min(hi, (1 << 64) - 1)))
        p.load(all_keys[sel], table[torch.from_numpy(sel)])
    ids = np.minimum((rng.pareto(1.2, rows * z) * 3).astype(np.int64), n_feat - 1).astype(np.int32)
    y = np.where(rng.random(rows) < 0.5, 1.0, -1.0).astype(np.float32)
    b = LocalBatch(rows, rows * z, S, "cuda")
    b.localize(torch.from_numpy(ids).cuda(), torch.from_numpy(y).cuda(), planes[0].bounds, fixed_z=z, hash_seed=11)
    ctx = (torch.randn(N, 64) * 0.3).to(torch.bfloat16).cuda()
    torch.cuda.synchronize()
    return planes, b, ctx, table, known, all_keys, ids, y, rows, z


@pytest.mark.parametrize("S,N", [(1, 64), (2, 128), (1, 128)])
def test_wide_pull_gemm_matches_fp32_matmul(cuda_lib, S, N):
    planes, b, ctx, table, known, all_keys, ids, y, rows, z = _setup(S, N)
    U = int(b.n_unique.item())
    P = torch.zeros(b.max_nnz, N, device="cuda")
    V = torch.zeros(b.max_nnz, 64, dtype=torch.bfloat16, device="cuda")
    planes[0].pull_gemm(b, ctx, P, V)
    torch.cuda.synchronize()
    planes[0].check_status()
    uk = b.ukeys[:U].cpu().numpy().view(np.uint64)
    idx = {int(k): i for i, k in enumerate(all_keys.tolist())}
    rows_ref = torch.stack([table[idx[int(k)]] if known[idx[int(k)]] else torch.zeros(64, dtype=torch.bfloat16) for k in uk.tolist()])
    assert torch.equal(V[:U].cpu(), rows_ref)                                  # the gather is exact
    ref = rows_ref.float() @ ctx.cpu().float().T
    assert torch.allclose(P[:U].cpu(), ref, rtol=1e-3, atol=1e-3), float((P[:U].cpu() - ref).abs().max())


@pytest.mark.parametrize("n_rows,fused", [(300, False), (900, False), (900, True)])
def test_wide_training_step_matches_reference(cuda_lib, n_rows, fused):
    """With 900 rows the most frequent key owns about 3,000 nonzeros: its gradient is
    reduced by several warps (segments above 256 nonzeros are split into chunks).
    ``fused``: the pull kernel adds the products into the rows' margins itself and no
    product matrix is stored."""
    S, N = 2, 64
    planes, b, ctx, table, known, all_keys, ids, y, rows, z = _setup(S, N, rows=n_rows, seed=4)
    assert int((b.seg_off[1:int(b.n_unique.item()) + 1] - b.seg_off[:int(b.n_unique.item())]).max().item()) > (256 if n_rows == 900 else 0)
    U = int(b.n_unique.item())
    w = planes[0]
    P = torch.zeros(b.max_nnz, N, device="cuda")
    if fused:
        w.pull_gemm(b, ctx, None, fuse_margins=True)
        w.rowloss(b)
    else:
        w.pull_gemm(b, ctx, P)
        w.rowsum(b, P, N)
    w.push(b, ctx, 0)
    # the other (virtual) worker pushes nothing: publish an empty round for it
    from parameter_server_b200.ops.localize import LocalBatch
    empty = LocalBatch(4, 16, S, "cuda")
    empty.n_unique.zero_(); empty.own_off.zero_(); empty.seg_off.zero_()
    planes[1].push(empty, ctx, 0)
    for p in planes:
        p.apply(0)
    torch.cuda.synchronize()
    for p in planes:
        p.check_status()
    # reference in fp32
    idx = {int(k): i for i, k in enumerate(all_keys.tolist())}
    uk = b.ukeys[:U].cpu().numpy().view(np.uint64)
    col = b.csr_col[:rows * z].cpu().numpy().reshape(rows, z)
    Vref = torch.stack([table[idx[int(k)]].float() if known[idx[int(k)]] else torch.zeros(64) for k in uk.tolist()])
    Pref = Vref @ ctx.cpu().float().T
    n_of_row = np.arange(rows) % N
    margin = Pref[torch.from_numpy(col), torch.from_numpy(n_of_row)[:, None]].sum(1)
    assert torch.allclose(b.margin[:rows].cpu(), margin, rtol=2e-3, atol=2e-3)
    ym = torch.from_numpy(y) * margin
    gcoef = -torch.from_numpy(y) * torch.sigmoid(-ym)
    assert torch.allclose(b.gcoef[:rows].cpu(), gcoef, rtol=2e-3, atol=2e-3)
    G = torch.zeros(U, 64)
    C = ctx.cpu().float()
    for r in range(rows):
        for j in range(z):
            G[col[r, j]] += gcoef[r] * C[n_of_row[r]]
    Gb = G.to(torch.bfloat16).float()                        # gradients travel as bf16
    acc = Gb * Gb
    Wref = (Vref - 0.1 / (acc.sqrt() + 1.0) * Gb).to(torch.bfloat16)
    got = torch.zeros(U, 64, dtype=torch.bfloat16)
    for p in planes:
        lo, hi = p.bounds_host[p.rank], p.bounds_host[p.rank + 1]
        sel = (uk >= np.uint64(lo)) & (uk < np.uint64(min(hi, (1 << 64) - 1)))
        got[torch.from_numpy(sel)] = p.lookup(uk[sel])
    diff = (got.float() - Wref.float()).abs()
    assert float(diff.max()) < 0.02 and float((diff > 0.004).float().mean()) < 0.02


@pytest.mark.parametrize("S,N", [(1, 64), (2, 128), (3, 64)])
def test_wide_exchange_pull_matches_fp32_matmul(cuda_lib, S, N):
    """Exchange form of the pull (keys to the owners, rows back in bulk, tcgen05 product on
    the local copy), ranks emulated on one GPU: the three roles run as separate launches."""
    from parameter_server_b200.ops.localize import LocalBatch
    rows, z = 300, 12
    planes, b, ctx, table, known, all_keys, ids, y, rows, z = _setup(S, N, rows=rows, z=z, seed=5, pull_cap=rows * z)
    U = int(b.n_unique.item())
    batches = [b]
    for _ in range(1, S):
        e = LocalBatch(4, rows * z, S, "cuda")
        e.n_unique.zero_(); e.own_off.zero_(); e.seg_off.zero_()
        batches.append(e)
    Ps = [torch.zeros(rows * z, N, device="cuda") for _ in range(S)]
    for rnd in range(2):                                   # two rounds: both parities of the buffers
        for phase in (1, 2, 4):
            for p, bb, P in zip(planes, batches, Ps):
                # the second round also adds the products into the rows' margins (fused form)
                p.pull_xgemm(bb, ctx, P, rnd, phases=phase, wait_iters=1 << 12, fuse_margins=rnd == 1)
        if rnd == 1:
            planes[0].rowloss(b)               # the fused margins are complete after the long segments are added
        torch.cuda.synchronize()
        for p in planes:
            p.check_status()
        idx = {int(k): i for i, k in enumerate(all_keys.tolist())}
        uk = b.ukeys[:U].cpu().numpy().view(np.uint64)
        Vref = torch.stack([table[idx[int(k)]].float() if known[idx[int(k)]] else torch.zeros(64) for k in uk.tolist()])
        assert torch.equal(planes[0].pulled_rows(rnd, U).cpu().float(), Vref)
        Pref = Vref @ ctx.cpu().float().T
        assert torch.allclose(Ps[0][:U].cpu(), Pref, rtol=2e-3, atol=2e-3)
        if rnd == 1:
            col = b.csr_col[:rows * z].cpu().numpy().reshape(rows, z)
            n_of_row = np.arange(rows) % N
            margin = Pref[torch.from_numpy(col), torch.from_numpy(n_of_row)[:, None]].sum(1)
            assert torch.allclose(b.margin[:rows].cpu(), margin, rtol=2e-3, atol=2e-3)
        Ps[0].zero_()
