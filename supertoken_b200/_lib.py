"""ctypes binding of ``libstbpe.so`` (the C ABI declared in ``include/stbpe.h``).

There is no CPU fallback: if the library is missing or cannot be loaded the import of
the product path fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("STBPE_LIB", os.path.join(_HERE, "libstbpe.so"))

OK, E_BADARG, E_CAPACITY, E_TIMEOUT, E_CUDA, E_ID_OVERFLOW, E_STATE = range(7)
RUNNING, STOP_TARGET, STOP_NO_PAIRS, STOP_LOW_COUNT, STOP_ERROR = range(5)


class Config(ctypes.Structure):
    _fields_ = [("device", ctypes.c_int32), ("base_vocab", ctypes.c_int32),
                ("max_tokens", ctypes.c_int64), ("table_slots", ctypes.c_int64),
                ("max_merges", ctypes.c_int32), ("world_size", ctypes.c_int32),
                ("rank", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class State(ctypes.Structure):
    _fields_ = [("merges_done", ctypes.c_int32), ("stop_reason", ctypes.c_int32),
                ("live_tokens", ctypes.c_int64), ("table_keys", ctypes.c_int64),
                ("table_slots", ctypes.c_int64), ("device_error", ctypes.c_uint32),
                ("n_tiles", ctypes.c_int32), ("fixups", ctypes.c_int64), ("repacks", ctypes.c_int64), ("work_tiles", ctypes.c_int64), ("count_kernel_ms", ctypes.c_double),
                ("count_convert_ms", ctypes.c_double),
                ("tile_bytes_in", ctypes.c_int64), ("tile_bytes_out", ctypes.c_int64)]


# every symbol include/stbpe.h declares: name -> (restype, argtypes)
_vp, _i64, _i32, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int
_P = ctypes.POINTER
SIGNATURES = {
    "stbpe_create": (_int, [_P(_vp), _P(Config)]),
    "stbpe_destroy": (_int, [_vp]),
    "stbpe_last_error": (ctypes.c_char_p, [_vp]),
    "stbpe_version": (ctypes.c_char_p, []),
    "stbpe_reset": (_int, [_vp]),
    "stbpe_append_bytes": (_int, [_vp, _vp, _i64, _vp, _i64, _vp]),
    "stbpe_append_ids": (_int, [_vp, _vp, _i64, _vp, _i64, _vp]),
    "stbpe_count_initial": (_int, [_vp, _vp]),
    "stbpe_select_best": (_int, [_vp, _P(ctypes.c_uint64), _P(_i64), _P(_i64), _vp]),
    "stbpe_apply_merge": (_int, [_vp, _i32, _i32, _i32, _P(_i64), _vp]),
    "stbpe_train": (_int, [_vp, _i32, _vp]),
    "stbpe_train_timed": (_int, [_vp, _i32, _P(ctypes.c_float), _vp]),
    "stbpe_repack": (_int, [_vp, _int, _P(_int), _vp]),
    "stbpe_get_state": (_int, [_vp, _P(State), _vp]),
    "stbpe_get_merges": (_int, [_vp, _i32, _i32, _vp, _vp, _vp]),
    "stbpe_export_histogram": (_int, [_vp, _vp, _vp, _i64, _P(_i64), _vp]),
    "stbpe_export_ties": (_int, [_vp, _i64, _vp, _i64, _P(_i64), _vp]),
    "stbpe_export_stream": (_int, [_vp, _vp, _i64, _P(_i64), _vp]),
    "stbpe_mg_set_buffers": (_int, [_vp, _vp, _vp, _i64]),
    "stbpe_mg_drain_only": (_int, [_vp, _vp]),
    "stbpe_mg_count_local": (_int, [_vp, _vp]),
    "stbpe_mg_merge_local": (_int, [_vp, _vp]),
    "stbpe_mg_apply_inbox": (_int, [_vp, _vp]),
    "stbpe_mg_candidate": (_int, [_vp, _vp, _vp]),
    "stbpe_mg_commit": (_int, [_vp, _vp, _vp]),
    "stbpe_mg_nccl_unique_id": (_int, [_vp]),
    "stbpe_mg_nccl_init": (_int, [_vp, _vp, _i64]),
    "stbpe_mg_run": (_int, [_vp, _int, _int, _vp]),
    "stbpe_mg_peer_export": (_int, [_vp, _i64, _vp]),
    "stbpe_mg_peer_open": (_int, [_vp, _vp, _i32]),
    "stbpe_mg_peer_run": (_int, [_vp, _int, _int, _vp]),
    "stbpe_mg_peer_close": (_int, [_vp]),
    "stbpe_mg_peer_mailbox": (_int, [_vp, _vp]),
    "stbpe_mg_peer_set": (_int, [_vp, _vp, _i32]),
    "stbpe_mg_wide_export": (_int, [_vp, _vp]),
    "stbpe_mg_wide_open": (_int, [_vp, _vp, _i32]),
    "stbpe_mg_wide_block": (_int, [_vp, _vp]),
    "stbpe_mg_wide_set": (_int, [_vp, _vp, _i32]),
    "stbpe_mg_wide_pass1": (_int, [_vp, _P(_i32), _vp]),
    "stbpe_mg_wide_pass2": (_int, [_vp, _vp]),
    "stbpe_mg_wide_close": (_int, [_vp]),
    "stbpe_rows_count_pairs": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp]),
    "stbpe_rows_count_pairs_noalloc": (_int, [_vp, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp,
                                              ctypes.c_char_p, ctypes.c_size_t]),
    "stbpe_rows_apply_merge": (_int, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _vp, _vp]),
}

_lib = None


class LibraryMissing(ImportError):
    pass


def load() -> ctypes.CDLL:
    """Load the CUDA library; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m supertoken_b200.build` "
            "(nvcc, sm_100a).  There is no CPU fallback for the BPE merge loop.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError = header and library out of step
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
