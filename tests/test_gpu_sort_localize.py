"""Radix sort and minibatch localisation against NumPy."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand_keys(n, rng, skew=False, bits=64):
    if skew:
        ids = (rng.pareto(1.05, n) * 3).astype(np.uint64) % np.uint64(1 << 20)
        from parameter_server_b200.utils.oracle import hash_id_to_key
        k = hash_id_to_key(ids, 7)
    else:
        k = rng.integers(0, 1 << 63, n, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, n, dtype=np.uint64)
    if bits < 64:
        k = k >> np.uint64(64 - bits)
    return k


@pytest.mark.parametrize("n", [1, 31, 4096, 4097, 100_003, 1_500_000])
@pytest.mark.parametrize("skew", [False, True])
def test_sort_pairs_matches_numpy(cuda_lib, n, skew):
    from parameter_server_b200.ops.localize import sort_pairs
    rng = np.random.default_rng(n + skew)
    k = _rand_keys(n, rng, skew)
    kt = torch.from_numpy(k.view(np.int64)).cuda()
    sk, sv = sort_pairs(kt)
    torch.cuda.synchronize()
    order = np.argsort(k, kind="stable")
    assert np.array_equal(sk.cpu().numpy().view(np.uint64), k[order])
    assert np.array_equal(sv.cpu().numpy().astype(np.int64), order)  # stable => identical permutation


def test_sort_partial_bits_and_payload(cuda_lib):
    from parameter_server_b200.ops.localize import sort_pairs
    rng = np.random.default_rng(3)
    n = 50_000
    k = _rand_keys(n, rng, bits=26)
    pay = rng.integers(0, 1 << 31, n, dtype=np.int64).astype(np.int32)
    sk, sv = sort_pairs(torch.from_numpy(k.view(np.int64)).cuda(), torch.from_numpy(pay).cuda(), 0, 26)
    order = np.argsort(k, kind="stable")
    assert np.array_equal(sk.cpu().numpy().view(np.uint64), k[order])
    assert np.array_equal(sv.cpu().numpy(), pay[order])


@pytest.mark.parametrize("S", [1, 2, 8])
@pytest.mark.parametrize("fixed", [True, False])
def test_localize_matches_numpy(cuda_lib, S, fixed):
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.utils.range import Range, shard_bounds
    rng = np.random.default_rng(11 + S)
    rows, z = 700, 37
    if fixed:
        row_ptr = np.arange(rows + 1) * z
    else:
        lens = rng.integers(0, 2 * z, rows)
        row_ptr = np.concatenate([[0], np.cumsum(lens)])
    nnz = int(row_ptr[-1])
    keys = _rand_keys(nnz, rng, skew=True)
    vals = rng.random(nnz, dtype=np.float32)
    b = LocalBatch(rows, nnz, S, "cuda", real_values=True)
    bounds_h = shard_bounds(Range.all(), S)
    bounds = torch.tensor([x if x < (1 << 63) else x - (1 << 64) for x in bounds_h], dtype=torch.int64).cuda()
    ids = torch.from_numpy(keys.view(np.int64)).cuda()
    kw = dict(fixed_z=z) if fixed else dict(row_ptr=torch.from_numpy(row_ptr.astype(np.int32)).cuda())
    b.localize(ids, None, bounds, vals=torch.from_numpy(vals).cuda(), hash_seed=None, method="sort", **kw)
    torch.cuda.synchronize()
    u, inv, cnt = np.unique(keys, return_inverse=True, return_counts=True)
    U = int(b.n_unique.item())
    assert U == len(u)
    assert np.array_equal(b.ukeys[:U].cpu().numpy().view(np.uint64), u)
    assert np.array_equal(b.csr_col[:nnz].cpu().numpy(), inv)
    seg = b.seg_off[:U + 1].cpu().numpy()
    assert np.array_equal(np.diff(seg), cnt)
    # CSC rows/values: each segment lists the rows containing that key, in position order
    rows_of = np.repeat(np.arange(rows), np.diff(row_ptr))
    order = np.argsort(keys, kind="stable")
    assert np.array_equal(b.csc_row[:nnz].cpu().numpy(), rows_of[order])
    assert np.allclose(b.csc_val[:nnz].cpu().numpy(), vals[order])
    own = b.own_off.cpu().numpy()
    exp = [int(np.searchsorted(u, np.uint64(x))) for x in bounds_h[:-1]] + [U]
    assert list(own) == exp
    # head bitmap consistent with segment offsets
    fb = b.flagbits[:(nnz + 31) // 32].cpu().numpy().view(np.uint32)
    heads = np.zeros(nnz, dtype=bool); heads[seg[:-1]] = True
    bits = np.unpackbits(fb.view(np.uint8), bitorder="little")[:nnz].astype(bool)
    assert np.array_equal(bits, heads)
    wb = b.wordbase[:(nnz + 31) // 32].cpu().numpy()
    assert np.array_equal(wb, np.concatenate([[0], np.cumsum(heads)])[0:nnz:32])


def test_hash_on_device_matches_oracle(cuda_lib):
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.utils.oracle import hash_id_to_key
    rng = np.random.default_rng(5)
    ids = rng.integers(0, 1 << 26, 64 * 50, dtype=np.int64).astype(np.int32)
    b = LocalBatch(64, ids.size, 1, "cuda")
    bounds = torch.tensor([0, -1], dtype=torch.int64).cuda()
    b.localize(torch.from_numpy(ids).cuda(), None, bounds, fixed_z=50, hash_seed=9)
    U = int(b.n_unique.item())
    assert np.array_equal(b.ukeys[:U].cpu().numpy().view(np.uint64), np.unique(hash_id_to_key(ids, 9)))


def test_sort_skips_constant_digits_and_narrow_hash(cuda_lib):
    """Keys with 40 significant bits (top bits): the three low digit passes are
    skipped on the device, the result is still the stable sorted order; and the
    device hash with 40 bits matches the NumPy restatement."""
    from parameter_server_b200.ops.localize import LocalBatch, sort_pairs
    from parameter_server_b200.utils.oracle import hash_id_to_key
    rng = np.random.default_rng(8)
    ids = rng.integers(0, 1 << 26, 64 * 300, dtype=np.int64).astype(np.int32)
    k = hash_id_to_key(ids, 0, 40)
    sk, sv = sort_pairs(torch.from_numpy(k.view(np.int64)).cuda())
    order = np.argsort(k, kind="stable")
    assert np.array_equal(sk.cpu().numpy().view(np.uint64), k[order])
    assert np.array_equal(sv.cpu().numpy().astype(np.int64), order)
    # already sorted input with identical keys: every pass is skipped, payload = index
    same = torch.full((5000,), 77, dtype=torch.int64, device="cuda")
    sk2, sv2 = sort_pairs(same)
    assert torch.equal(sv2.cpu(), torch.arange(5000, dtype=torch.int32)) and torch.equal(sk2, same)
    b = LocalBatch(64, ids.size, 2, "cuda")
    bounds = torch.tensor([0, -(1 << 63), -1], dtype=torch.int64).cuda()
    b.localize(torch.from_numpy(ids).cuda(), None, bounds, fixed_z=300, hash_seed=0, hash_bits=40, method="sort")
    U = int(b.n_unique.item())
    u = np.unique(k)
    assert np.array_equal(b.ukeys[:U].cpu().numpy().view(np.uint64), u)
    assert b.own_off.cpu().tolist() == [0, int(np.searchsorted(u, np.uint64(1 << 63))), U]
    rows_of = np.repeat(np.arange(64), 300)
    assert np.array_equal(b.csc_row[:ids.size].cpu().numpy(), rows_of[order])


@pytest.mark.parametrize("hash_bits,rows,z", [(40, 512, 100), (48, 300, 37), (20, 200, 64)])
def test_packed_positions_match_pair_sort(cuda_lib, hash_bits, rows, z):
    """Narrow hashed keys: sorting (key | position) single words gives exactly the
    same localised batch as sorting (key, position) pairs."""
    from parameter_server_b200.ops.localize import LocalBatch
    rng = np.random.default_rng(31)
    ids = (rng.zipf(1.3, rows * z) % (1 << 22)).astype(np.int32)
    vals = rng.random(rows * z, dtype=np.float32)
    bounds = torch.tensor([0, 1 << 62, -(1 << 63), -1], dtype=torch.int64).cuda()
    out = []
    for packed in (True, False):
        b = LocalBatch(rows, ids.size, 3, "cuda", real_values=True)
        b.localize(torch.from_numpy(ids).cuda(), None, bounds, fixed_z=z, vals=torch.from_numpy(vals).cuda(),
                   hash_seed=3, hash_bits=hash_bits, key_bits=(64 - hash_bits, 64), packed=packed, method="sort")
        torch.cuda.synchronize()
        assert (b.pack_bits > 0) == packed
        U = int(b.n_unique.item())
        out.append((U, b.ukeys[:U].cpu(), b.seg_off[:U + 1].cpu(), b.csr_col[:ids.size].cpu(),
                    b.csc_row[:ids.size].cpu(), b.csc_val[:ids.size].cpu(), b.own_off.cpu(),
                    b.flagbits[:(ids.size + 31) // 32].cpu(), b.wordbase[:(ids.size + 31) // 32].cpu()))
    assert out[0][0] == out[1][0] and out[0][0] > 1
    for x, y in zip(out[0][1:], out[1][1:]):
        assert torch.equal(x, y)


def _check_grouped(b, keys, row_ptr, vals, bounds_h, rows):
    """Every output of a localised batch against NumPy, with the rows of a key's
    CSC segment compared as a set (the bucket path does not order them)."""
    nnz = keys.size
    u, inv, cnt = np.unique(keys, return_inverse=True, return_counts=True)
    U = int(b.n_unique.item())
    assert U == len(u)
    assert np.array_equal(b.ukeys[:U].cpu().numpy().view(np.uint64), u)
    assert np.array_equal(b.csr_col[:nnz].cpu().numpy(), inv)
    seg = b.seg_off[:U + 1].cpu().numpy().astype(np.int64)
    assert seg[0] == 0 and seg[-1] == nnz
    assert np.array_equal(np.diff(seg), cnt)
    rows_of = np.repeat(np.arange(rows), np.diff(row_ptr))
    order = np.argsort(keys, kind="stable")
    seg_id = np.repeat(np.arange(U), cnt)
    got_rows = b.csc_row[:nnz].cpu().numpy().astype(np.int64)
    exp_rows = rows_of[order]
    if vals is None:
        assert np.array_equal(np.sort(seg_id * (rows + 1) + got_rows), np.sort(seg_id * (rows + 1) + exp_rows))
    else:
        # (row, value) pairs per segment, as sets
        got_v = b.csc_val[:nnz].cpu().numpy()
        g = np.lexsort((got_v, got_rows, seg_id))
        e = np.lexsort((vals[order], exp_rows, seg_id))
        assert np.array_equal(got_rows[g], exp_rows[e])
        assert np.array_equal(got_v[g], vals[order][e])
    own = b.own_off.cpu().numpy()
    assert list(own) == [int(np.searchsorted(u, np.uint64(x))) for x in bounds_h[:-1]] + [U]
    fb = b.flagbits[:(nnz + 31) // 32].cpu().numpy().view(np.uint32)
    heads = np.zeros(nnz, dtype=bool); heads[seg[:-1]] = True
    bits = np.unpackbits(fb.view(np.uint8), bitorder="little")[:nnz].astype(bool)
    assert np.array_equal(bits, heads)
    wb = b.wordbase[:(nnz + 31) // 32].cpu().numpy()
    assert np.array_equal(wb, np.concatenate([[0], np.cumsum(heads)])[0:nnz:32])


def _bounds(S):
    from parameter_server_b200.utils.range import Range, shard_bounds
    bounds_h = shard_bounds(Range.all(), S)
    return bounds_h, torch.tensor([x if x < (1 << 63) else x - (1 << 64) for x in bounds_h], dtype=torch.int64).cuda()


@pytest.mark.parametrize("hash_bits,rows,z,S", [(40, 2048, 100, 1), (40, 4096, 200, 8), (0, 1500, 64, 3), (52, 700, 37, 2)])
def test_bucket_localize_hashed_ids(cuda_lib, hash_bits, rows, z, S):
    """Bucket path on device-hashed ids with a heavy head (frequent keys go through
    the counting path, the rest through the per-bucket tables)."""
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.utils.oracle import hash_id_to_key
    rng = np.random.default_rng(hash_bits + rows)
    ids = (rng.zipf(1.2, rows * z) % (1 << 24)).astype(np.int32)
    keys = hash_id_to_key(ids, 5, hash_bits or 64)
    bounds_h, bounds = _bounds(S)
    b = LocalBatch(rows, ids.size, S, "cuda")
    b.localize(torch.from_numpy(ids).cuda(), None, bounds, fixed_z=z, hash_seed=5, hash_bits=hash_bits, method="bucket")
    torch.cuda.synchronize()
    assert int(b.gate.item()) == 0, "the bucket path gave up on evenly spread keys"
    assert int(b.status.item()) == 0
    _check_grouped(b, keys, np.arange(rows + 1) * z, None, bounds_h, rows)


def test_bucket_localize_raw_keys_rows_and_values(cuda_lib):
    """Raw 64-bit keys (no device hash, positions in their own array), CSR row
    offsets and real values."""
    from parameter_server_b200.ops.localize import LocalBatch
    rng = np.random.default_rng(77)
    rows = 3000
    lens = rng.integers(0, 60, rows)
    row_ptr = np.concatenate([[0], np.cumsum(lens)])
    nnz = int(row_ptr[-1])
    keys = _rand_keys(nnz, rng, skew=True)
    vals = rng.random(nnz, dtype=np.float32)
    bounds_h, bounds = _bounds(4)
    b = LocalBatch(rows, nnz, 4, "cuda", real_values=True)
    b.localize(torch.from_numpy(keys.view(np.int64)).cuda(), None, bounds,
               row_ptr=torch.from_numpy(row_ptr.astype(np.int32)).cuda(), vals=torch.from_numpy(vals).cuda(),
               hash_seed=None, method="bucket")
    torch.cuda.synchronize()
    assert int(b.gate.item()) == 0 and int(b.status.item()) == 0
    _check_grouped(b, keys, row_ptr, vals, bounds_h, rows)


def test_bucket_localize_all_distinct_and_all_equal(cuda_lib):
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.utils.oracle import hash_id_to_key
    bounds_h, bounds = _bounds(2)
    rows, z = 1024, 64
    for ids in (np.arange(rows * z, dtype=np.int32), np.full(rows * z, 12345, dtype=np.int32)):
        keys = hash_id_to_key(ids, 1, 40)
        b = LocalBatch(rows, ids.size, 2, "cuda")
        b.localize(torch.from_numpy(ids).cuda(), None, bounds, fixed_z=z, hash_seed=1, hash_bits=40, method="bucket")
        torch.cuda.synchronize()
        assert int(b.gate.item()) == 0 and int(b.status.item()) == 0
        _check_grouped(b, keys, np.arange(rows + 1) * z, None, bounds_h, rows)


def test_auto_falls_back_to_sort_on_clustered_keys(cuda_lib):
    """Small integer keys all fall into the first bucket: the bucket path raises its
    flag on the device and the gated sort path produces the result."""
    from parameter_server_b200.ops.localize import LocalBatch
    rng = np.random.default_rng(9)
    rows, z = 2000, 50
    keys = rng.integers(1, 200_000, rows * z, dtype=np.int64).astype(np.uint64)
    bounds_h, bounds = _bounds(2)
    b = LocalBatch(rows, keys.size, 2, "cuda")
    b.localize(torch.from_numpy(keys.view(np.int64)).cuda(), None, bounds, fixed_z=z, hash_seed=None, method="auto")
    torch.cuda.synchronize()
    assert int(b.gate.item()) == 1 and int(b.status.item()) == 0
    _check_grouped(b, keys, np.arange(rows + 1) * z, None, bounds_h, rows)
    # the same buffers, next minibatch with spread keys: the bucket path runs again
    keys2 = _rand_keys(rows * z, rng, skew=True)
    b.localize(torch.from_numpy(keys2.view(np.int64)).cuda(), None, bounds, fixed_z=z, hash_seed=None, method="auto")
    torch.cuda.synchronize()
    assert int(b.gate.item()) == 0 and int(b.status.item()) == 0
    _check_grouped(b, keys2, np.arange(rows + 1) * z, None, bounds_h, rows)
