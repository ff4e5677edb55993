"""Ids as a bit stream: the NumPy packer against its inverse, and (on a GPU) the device unpacker."""
import numpy as np
import pytest

from parameter_server_b200.utils.idpack import bits_for, pack_ids, unpack_ids


@pytest.mark.parametrize("bits,n", [(26, 1000), (26, 33), (1, 70), (32, 100), (17, 12345), (5, 1)])
def test_pack_then_unpack_is_identity(bits, n):
    ids = np.random.default_rng(bits * 1000 + n).integers(0, 1 << bits, n, dtype=np.uint64)
    words = pack_ids(ids, bits)
    assert words.dtype == np.uint32 and words.size % 4 == 0 and words.size * 32 >= n * bits + 32
    assert np.array_equal(unpack_ids(words, bits, n), ids.astype(np.uint32))


def test_bits_for_and_overflow_is_refused():
    assert bits_for((1 << 26) - 1) == 26 and bits_for(1 << 26) == 27 and bits_for(0) == 1
    with pytest.raises(AssertionError):
        pack_ids(np.array([8], dtype=np.uint64), 3)


@pytest.mark.gpu
def test_device_unpack_and_localize_from_packed_ids(cuda_lib):
    import torch
    from parameter_server_b200.ops import _lib as L
    from parameter_server_b200.ops.localize import LocalBatch
    from parameter_server_b200.utils.idpack import PackedIds
    rng = np.random.default_rng(1)
    rows, z, bits = 700, 16, 21
    ids = rng.integers(0, 1 << bits, rows * z, dtype=np.uint64)
    pk = PackedIds.from_ids(ids, bits)
    dev_pk = PackedIds(pk.words.cuda(), pk.bits, pk.n)
    out = torch.empty(pk.n, dtype=torch.int32, device="cuda")
    L.check(L.lib().psb_unpack_ids(L.ptr(dev_pk.words), bits, pk.n, L.ptr(out), L.stream_ptr()), "unpack")
    assert np.array_equal(out.cpu().numpy().astype(np.uint32), ids.astype(np.uint32))
    # the localisation of the packed form equals that of the plain int32 ids
    y = torch.ones(rows, device="cuda")
    bounds = torch.tensor([0, -1], dtype=torch.int64, device="cuda")
    a, b = LocalBatch(rows, rows * z, 1, "cuda"), LocalBatch(rows, rows * z, 1, "cuda")
    a.localize(torch.from_numpy(ids.astype(np.int32)).cuda(), y, bounds, fixed_z=z, hash_seed=3)
    b.localize(dev_pk, y, bounds, fixed_z=z, hash_seed=3)
    torch.cuda.synchronize()
    U = int(a.n_unique.item())
    assert U == int(b.n_unique.item())
    assert torch.equal(a.ukeys[:U], b.ukeys[:U]) and torch.equal(a.seg_off[:U + 1], b.seg_off[:U + 1])
    assert torch.equal(a.csr_col[:rows * z], b.csr_col[:rows * z])
