"""ctypes binding of ``libpsb_cuda.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`parameter_server_b200._build`. Loading is
lazy; on a machine with a GPU a missing or unloadable library is an error (no
silent PyTorch fallback), on a CPU-only machine :func:`available` is False.

Every launcher returns 0 or minus a ``cudaError``; :func:`check` turns that into
an exception. ``LAUNCHES`` counts kernel launchers called through this module,
which is what the benchmarks report as the number of own-kernel launches.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

MAX_SHARDS = 16
ALGO_FTRL, ALGO_ADAGRAD, ALGO_SGD, ALGO_SUM, ALGO_KEEP = 0, 1, 2, 3, 4
LR_CONSTANT, LR_DECAY = 0, 1
LOSS_LOGIT, LOSS_SQUARE_HINGE = 0, 1
QUANT_NONE, QUANT_INT8, QUANT_FP16 = 0, 1, 2

STATUS_NAMES = {
    0: "ok", 1: "table full", 2: "inbox overflow", 3: "flag wait timed out",
    4: "grid barrier timed out", 5: "look-back timed out", 6: "bad argument",
}

_vp, _u32, _u64, _i32, _f32, _f64 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float, C.c_double


class Optimizer(C.Structure):
    _fields_ = [("algo", _i32), ("lr_type", _i32), ("alpha", _f32), ("beta", _f32),
                ("l1", _f32), ("l2", _f32)]


class PullParams(C.Structure):
    _fields_ = [
        ("S", _i32), ("insert", _i32),
        ("table", _vp * MAX_SHARDS), ("mask", _u64 * MAX_SHARDS),
        ("key_begin", _u64 * MAX_SHARDS), ("slot_mult", _u64 * MAX_SHARDS), ("applied", _vp * MAX_SHARDS),
        ("need_applied", _u32),
        ("ukeys", _vp), ("n_unique", _vp), ("own_off", _vp),
        ("w_local", _vp), ("slot_local", _vp), ("key_hit", _vp), ("grad_zero", _vp),
        ("row_ptr", _vp), ("n_rows", _u32), ("fixed_z", _u32),
        ("csr_col", _vp), ("csr_val", _vp), ("y", _vp), ("loss", _i32),
        ("gcoef", _vp), ("margin", _vp), ("stats", _vp), ("auc_hist", _vp),
        ("bar", _vp), ("status", _vp),
    ]


class PullExchangeParams(C.Structure):
    _fields_ = [
        ("S", _i32), ("me", _i32), ("ts1", _u32), ("need_applied", _u32), ("req_cap", _u32), ("wait_iters", _u32),
        ("phases", _i32),
        ("req_keys", _vp * MAX_SHARDS), ("req_hdr", _vp * MAX_SHARDS), ("req_ready", _vp * MAX_SHARDS),
        ("my_req_keys", _vp * MAX_SHARDS), ("my_req_hdr", _vp * MAX_SHARDS), ("my_req_ready", _vp * MAX_SHARDS),
        ("resp_w", _vp * MAX_SHARDS), ("resp_ready", _vp * MAX_SHARDS), ("slot_cache", _vp * MAX_SHARDS),
        ("alive", C.c_uint8 * MAX_SHARDS),
        ("table", _vp), ("mask", _u64), ("key_begin", _u64), ("slot_mult", _u64), ("applied", _vp),
        ("my_resp_w", _vp), ("my_resp_ready", _vp * MAX_SHARDS),
        ("ukeys", _vp), ("n_unique", _vp), ("own_off", _vp), ("grad_zero", _vp),
        ("row_ptr", _vp), ("n_rows", _u32), ("fixed_z", _u32), ("csr_col", _vp), ("csr_val", _vp), ("y", _vp),
        ("loss", _i32), ("gcoef", _vp), ("margin", _vp), ("stats", _vp), ("auc_hist", _vp),
        ("done", _vp), ("status", _vp),
        ("key_cache", _i32), ("kc_state", _vp), ("bar", _vp), ("slot_cache_prev", _vp * MAX_SHARDS),
        ("width", _i32), ("wide_vals", _vp),
        ("tile_off", _vp), ("tile_off_prev", _vp), ("tiles", _i32), ("key_end", _u64),
    ]


class PushParams(C.Structure):
    _fields_ = [
        ("S", _i32), ("ts1", _u32), ("inbox_cap", _u32), ("quant", _i32), ("send_keys", _i32),
        ("key_hit", _vp), ("mode", _vp * MAX_SHARDS),
        ("inbox_keys", _vp * MAX_SHARDS), ("inbox_vals", _vp * MAX_SHARDS),
        ("ready", _vp * MAX_SHARDS), ("count", _vp * MAX_SHARDS), ("applied", _vp * MAX_SHARDS),
        ("need_applied", _u32),
        ("ukeys", _vp), ("n_unique", _vp), ("own_off", _vp),
        ("nnz", _u32), ("csc_row", _vp), ("csc_val", _vp), ("flagbits", _vp), ("wordbase", _vp),
        ("gcoef", _vp), ("grad", _vp), ("bar", _vp), ("done", _vp), ("status", _vp),
        ("width", _i32),
    ]


class ApplyParams(C.Structure):
    _fields_ = [
        ("S", _i32), ("ts1", _u32), ("inbox_cap", _u32), ("quant", _i32),
        ("table", _vp), ("mask", _u64), ("key_begin", _u64), ("slot_mult", _u64),
        ("inbox_keys", _vp * MAX_SHARDS), ("inbox_vals", _vp * MAX_SHARDS),
        ("ready", _vp * MAX_SHARDS), ("count", _vp * MAX_SHARDS),
        ("alive", C.c_uint8 * MAX_SHARDS), ("cached", C.c_uint8 * MAX_SHARDS),
        ("mode", _vp * MAX_SHARDS),
        ("slot_cache", _vp * MAX_SHARDS),
        ("opt", Optimizer), ("stats", _vp), ("applied", _vp), ("wait_iters", _u32),
        ("bar", _vp), ("done", _vp), ("status", _vp),
        ("width", _i32), ("wide_vals", _vp),
        ("tile_off", _vp), ("tiles", _i32), ("slow", _vp),
    ]


class DarlinGrad(C.Structure):
    _fields_ = [
        ("S", _i32), ("ts1", _u32), ("c0", _u32), ("c1", _u32), ("u0", _u32), ("u1", _u32), ("block_cap", _u32),
        ("shard_col", _u32 * (MAX_SHARDS + 1)),
        ("seg_off", _vp), ("csc_row", _vp), ("csc_val", _vp), ("flagbits", _vp), ("wordbase", _vp), ("gcol", _vp),
        ("y", _vp), ("margin", _vp), ("active", _vp), ("delta", _vp), ("stage", _vp),
        ("gu_inbox", _vp * MAX_SHARDS), ("ready", _vp * MAX_SHARDS),
        ("bar", _vp), ("done", _vp), ("status", _vp), ("csc_col", _vp), ("nz0", _u32), ("nz1", _u32),
    ]


class DarlinUpdate(C.Structure):
    _fields_ = [
        ("S", _i32), ("ts1", _u32), ("c0", _u32), ("c1", _u32), ("my0", _u32), ("my1", _u32), ("block_cap", _u32),
        ("gu_inbox", _vp * MAX_SHARDS), ("ready", _vp * MAX_SHARDS), ("alive", C.c_uint8 * MAX_SHARDS),
        ("w", _vp), ("delta", _vp), ("active", _vp),
        ("eta", _f32), ("lam", _f32), ("delta_max", _f32), ("kkt_threshold", _f32),
        ("wnew_inbox", _vp * MAX_SHARDS), ("wnew_ready", _vp * MAX_SHARDS),
        ("violation", _vp), ("wait_iters", _u32), ("done", _vp), ("status", _vp),
    ]


class DarlinDual(C.Structure):
    _fields_ = [
        ("S", _i32), ("ts1", _u32), ("c0", _u32), ("c1", _u32), ("u0", _u32), ("u1", _u32), ("block_cap", _u32),
        ("shard_col", _u32 * (MAX_SHARDS + 1)),
        ("seg_off", _vp), ("csc_row", _vp), ("csc_val", _vp), ("flagbits", _vp), ("wordbase", _vp), ("gcol", _vp),
        ("margin", _vp), ("w_cur", _vp), ("delta", _vp), ("active", _vp), ("delta_max", _f32),
        ("wnew", _vp), ("wnew_ready", _vp * MAX_SHARDS), ("alive", C.c_uint8 * MAX_SHARDS),
        ("wait_iters", _u32), ("bar", _vp), ("status", _vp), ("csc_col", _vp), ("nz0", _u32), ("nz1", _u32),
    ]


class DarlinPass(C.Structure):
    _fields_ = [
        ("grad", _vp), ("update", _vp), ("dual", _vp), ("order", _vp),
        ("n_steps", _u32), ("ts_base", _u32), ("tau", _i32), ("ring", _i32),
        ("kkt_threshold", _f32), ("wait_iters", _u32), ("bar", _vp), ("status", _vp),
        ("phase_ns", _vp),
    ]


_LIB = None
LAUNCHES = 0


def lib_path() -> Path:
    """The in-tree CUDA library; ``PSB_CUDA_LIB`` selects another build of it (e.g. one with tracing)."""
    override = os.environ.get("PSB_CUDA_LIB")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent.parent / "libpsb_cuda.so"


def available() -> bool:
    return torch.cuda.is_available() and lib_path().exists()


def _declare(lib):
    sz = C.c_size_t
    lib.psb_sort_scratch_bytes.restype = sz
    lib.psb_sort_scratch_bytes.argtypes = [_u32, _i32, _i32]
    lib.psb_sort_pairs.argtypes = [_vp, _i32, _u64, _vp, _vp, _i32, _vp, _vp, _u32, _i32, _i32, _vp, _vp, _vp, _i32, _vp]
    lib.psb_localize2.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _vp, _u32, _u32, _vp, _vp, _i32, _vp, _vp, _vp, _vp,
                                  _vp, _vp, _vp, _vp, _vp, _i32, _vp]
    lib.psb_owner_offsets.argtypes = [_vp, _vp, _vp, _i32, _vp, _vp]
    lib.psb_sort_pairs_gated.argtypes = [_vp, _i32, _u64, _vp, _vp, _i32, _vp, _vp, _u32, _i32, _i32, _vp, _vp, _vp, _i32,
                                         _vp, _vp]
    lib.psb_localize2_gated.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _vp, _u32, _u32, _vp, _vp, _i32, _vp, _vp, _vp,
                                        _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp]
    lib.psb_bucket_localize_scratch_bytes.restype = sz
    lib.psb_bucket_localize_scratch_bytes.argtypes = [_u32]
    lib.psb_bucket_localize.argtypes = [_vp, _i32, _u64, _u32, _i32, _vp, _u32, _u32, _vp, _vp, _i32, _vp, _vp, _vp,
                                        _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]
    lib.psb_localize_scratch_bytes.restype = sz
    lib.psb_localize_scratch_bytes.argtypes = [_u32]
    lib.psb_localize.argtypes = [_vp, _vp, _u32, _vp, _u32, _u32, _vp, _vp, _i32, _vp, _vp, _vp, _vp,
                                 _vp, _vp, _vp, _vp, _vp, _vp]
    lib.psb_table_init.argtypes = [_vp, _u64, _vp]
    lib.psb_pull_margin.argtypes = [C.POINTER(PullParams), _vp]
    lib.psb_push.argtypes = [C.POINTER(PushParams), _vp]
    lib.psb_pull_exchange.argtypes = [C.POINTER(PullExchangeParams), _vp]
    lib.psb_apply.argtypes = [C.POINTER(ApplyParams), _vp]
    lib.psb_table_dump.argtypes = [_vp, _u64, _vp, _vp, _u64, _vp, _vp]
    lib.psb_table_load.argtypes = [_vp, _u64, _u64, _u64, _vp, _vp, _vp, _vp, _u64, _vp, _vp]
    lib.psb_table_export.argtypes = [_vp, _u64, _vp, _vp, _vp, _vp, _u64, _vp, _vp]
    lib.psb_coop_grid.argtypes = [_i32]
    lib.psb_darlin_grad.argtypes = [C.POINTER(DarlinGrad), _vp]
    lib.psb_darlin_update.argtypes = [C.POINTER(DarlinUpdate), _vp]
    lib.psb_darlin_dual.argtypes = [C.POINTER(DarlinDual), _vp]
    lib.psb_darlin_pass.argtypes = [C.POINTER(DarlinPass), _vp]
    lib.psb_darlin_eval.argtypes = [_vp, _vp, _u32, _vp, _vp, _u32, _u32, _f32, _vp, _vp]
    lib.psb_darlin_struct_size.argtypes = [_i32]
    lib.psb_key_signature.argtypes = [_vp, _vp, _u32, _vp, _vp, _vp, _vp, _vp]
    lib.psb_fixfloat_encode.argtypes = [_vp, _vp, _u64, _i32, _f32, _f32, _u64, _vp]
    lib.psb_fixfloat_decode.argtypes = [_vp, _vp, _u64, _i32, _f32, _f32, _vp]
    lib.psb_minmax.argtypes = [_vp, _u64, _vp, _vp]
    lib.psb_add_noise.argtypes = [_vp, _u64, _f32, _f32, _u64, _vp]
    lib.psb_countmin_insert.argtypes = [_vp, _u32, _i32, _vp, _vp, _vp, _u32, _vp]
    lib.psb_countmin_query.argtypes = [_vp, _u32, _i32, _vp, _vp, _vp, _u32, _vp]
    lib.psb_ordered_match.argtypes = [_vp, _vp, _u32, _vp, _vp, _u32, _i32, _i32, _vp, _vp]
    lib.psb_gen_batch.argtypes = [_vp, _vp, _vp, _vp, _u32, _u32, _u64, _f64, _u64, _u64, _i32, _vp]
    lib.psb_hash_ids.argtypes = [_vp, _vp, _vp, _u64, _u64, _vp]
    lib.psb_flush_l2.argtypes = [_vp, _u64, _u32, _vp]
    lib.psb_unpack_ids.argtypes = [_vp, _i32, _u32, _vp, _vp]
    lib.psb_heap_alloc.argtypes = [C.POINTER(_vp), sz]
    lib.psb_heap_free.argtypes = [_vp]
    lib.psb_ipc_export.argtypes = [_vp, _vp]
    lib.psb_ipc_open.argtypes = [_vp, C.POINTER(_vp)]
    lib.psb_ipc_close.argtypes = [_vp]
    lib.psb_set_device.argtypes = [_i32]
    lib.psb_can_access_peer.argtypes = [_i32, _i32]
    lib.psb_error_string.restype = C.c_char_p
    lib.psb_error_string.argtypes = [_i32]
    for name, proto in _EXTRA_PROTOS.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            if proto[0] is not None:
                fn.restype = proto[0]
            fn.argtypes = proto[1]


# prototypes registered by other op modules (filters, darlin, wide, ...)
_EXTRA_PROTOS: dict = {}


def register_protos(protos: dict):
    _EXTRA_PROTOS.update(protos)
    if _LIB is not None:
        _declare(_LIB)


def lib():
    """The loaded CUDA library. Raises if it cannot be loaded."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: run `python -m parameter_server_b200._build` "
                "(or __graft_entry__.build()) first")
        _LIB = C.CDLL(os.fspath(path), mode=C.RTLD_GLOBAL)
        _declare(_LIB)
        for which, st in enumerate((PullParams, PushParams, ApplyParams, Optimizer, PullExchangeParams)):
            if _LIB.psb_struct_size(which) != C.sizeof(st):
                raise RuntimeError(f"{st.__name__}: binding struct is {C.sizeof(st)} bytes, "
                                   f"library expects {_LIB.psb_struct_size(which)}")
        for which, st in enumerate((DarlinGrad, DarlinUpdate, DarlinDual, DarlinPass)):
            if _LIB.psb_darlin_struct_size(which) != C.sizeof(st):
                raise RuntimeError(f"{st.__name__}: binding struct is {C.sizeof(st)} bytes, "
                                   f"library expects {_LIB.psb_darlin_struct_size(which)}")
    return _LIB


class PsbCudaError(RuntimeError):
    pass


def check(rc: int, what: str = "", kernels: int = 1) -> int:
    """Raise on a negative launcher return code; count ``kernels`` launches."""
    global LAUNCHES
    LAUNCHES += kernels
    if rc < 0:
        msg = lib().psb_error_string(rc).decode()
        raise PsbCudaError(f"{what or 'psb'} failed: {msg} ({-rc})")
    return rc


def ptr(t) -> int:
    """Device address of a tensor (0 for None)."""
    if t is None:
        return 0
    return t.data_ptr()


def stream_ptr(stream=None) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream


def check_status(status: torch.Tensor, what: str = "", reset=()):
    """Host check of a device status word (synchronises). On an error the status word and the
    tensors in ``reset`` are zeroed before the exception is raised: a kernel that gave up at a grid
    barrier leaves its barrier and arrival counters half counted, and with them every later launch
    would fail the same way; zeroed, the object that owns them can be used again."""
    code = int(status.item())
    if code != 0:
        if status.is_cuda:
            torch.cuda.synchronize(status.device)      # every stream: nothing may still count on those words
        status.zero_()
        for t in reset:
            if t is not None:
                t.zero_()
        raise PsbCudaError(f"{what or 'kernel'} reported status {code}: {STATUS_NAMES.get(code, '?')}")
