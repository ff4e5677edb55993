"""The allocation-free localise entry point against the regular one.

`psb_localize_static` is for embedders that cannot allocate device memory at
call time (all free memory already handed to their own pool, a loop that must
not touch the allocator, a plug-in without an allocator handle): its scratch is a
fixed array inside the library. It is called here through its exported C symbol,
twice in a row (the scratch keeps the first call's contents), and every output
must equal what `psb_localize` produces from the same input. Inputs larger than
the built-in scratch must be refused without launching anything.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_N = 16 * 1024 * 1024


def _outputs(nnz, S, dev):
    i32, i64 = torch.int32, torch.int64
    return dict(ukeys=torch.zeros(nnz, dtype=i64, device=dev), seg_off=torch.zeros(nnz + 1, dtype=i32, device=dev),
                csr_col=torch.zeros(nnz, dtype=i32, device=dev), flagbits=torch.zeros((nnz + 31) // 32, dtype=i32, device=dev),
                wordbase=torch.zeros((nnz + 31) // 32, dtype=i32, device=dev), n_unique=torch.zeros(1, dtype=i32, device=dev),
                own_off=torch.zeros(S + 1, dtype=i32, device=dev))


def test_static_scratch_entry_point_matches_regular_one(cuda_lib):
    from parameter_server_b200.ops._lib import ptr, stream_ptr
    from parameter_server_b200.ops.localize import sort_pairs
    L = cuda_lib
    vp, u32 = C.c_void_p, C.c_uint32
    fn = L.psb_localize_static                      # the exported C symbol
    fn.restype = C.c_int
    fn.argtypes = [vp, vp, u32, vp, u32, u32, vp, vp, C.c_int] + [vp] * 8 + [vp]
    dev = torch.device("cuda")
    S = 4
    bounds = torch.tensor([0, 1 << 62, (1 << 63) - (1 << 64), -(1 << 62), -1], dtype=torch.int64, device=dev)
    rng = np.random.default_rng(0)
    for call, (rows, z) in enumerate([(3000, 40), (777, 13)]):     # two calls in a row, different sizes
        nnz = rows * z
        ids = np.minimum((rng.pareto(1.05, nnz) * 5).astype(np.int64), 50_000)
        keys = (ids.astype(np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        sk, sp = sort_pairs(torch.from_numpy(keys.view(np.int64)).to(dev))
        ref, got = _outputs(nnz, S, dev), _outputs(nnz, S, dev)
        pos_ref, pos_got = sp.clone(), sp.clone()
        scratch = torch.empty(L.psb_localize_scratch_bytes(nnz), dtype=torch.uint8, device=dev)
        rc = L.psb_localize(ptr(sk), ptr(pos_ref), nnz, 0, rows, z, 0, ptr(bounds), S, ptr(ref["ukeys"]),
                            ptr(ref["seg_off"]), ptr(ref["csr_col"]), 0, ptr(ref["flagbits"]), ptr(ref["wordbase"]),
                            ptr(ref["n_unique"]), ptr(ref["own_off"]), ptr(scratch), stream_ptr())
        assert rc == 0
        rc = fn(ptr(sk), ptr(pos_got), nnz, 0, rows, z, 0, ptr(bounds), S, ptr(got["ukeys"]), ptr(got["seg_off"]),
                ptr(got["csr_col"]), 0, ptr(got["flagbits"]), ptr(got["wordbase"]), ptr(got["n_unique"]),
                ptr(got["own_off"]), stream_ptr())
        assert rc == 0, f"call {call} failed with {rc}"
        torch.cuda.synchronize()
        U = int(ref["n_unique"].item())
        assert int(got["n_unique"].item()) == U and U == len(np.unique(keys))
        assert torch.equal(got["ukeys"][:U], ref["ukeys"][:U])
        assert torch.equal(got["seg_off"][:U + 1], ref["seg_off"][:U + 1])
        for name in ("csr_col", "flagbits", "wordbase", "own_off"):
            assert torch.equal(got[name], ref[name]), name
        assert torch.equal(pos_got, pos_ref)            # positions rewritten to CSC row ids
    # beyond the built-in scratch: refused, nothing launched
    rc = fn(ptr(sk), ptr(pos_got), MAX_N + 1, 0, rows, z, 0, ptr(bounds), S, ptr(got["ukeys"]), ptr(got["seg_off"]),
            ptr(got["csr_col"]), 0, ptr(got["flagbits"]), ptr(got["wordbase"]), ptr(got["n_unique"]),
            ptr(got["own_off"]), stream_ptr())
    assert rc == -1                                     # cudaErrorInvalidValue
    torch.cuda.synchronize()
