"""ctypes binding of ``libshmt.so`` — the only way Python reaches the CUDA code.

The library is looked for next to this file.  There is no fallback of any
kind: if it is missing the import fails with the build command to run.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# SHMT_LIBRARY points at another build of the same library (a tuning variant); default: in-tree
LIB_PATH = Path(os.environ.get("SHMT_LIBRARY") or Path(__file__).resolve().parent / "libshmt.so")

OK, ERR_INVALID, ERR_CUDA, ERR_CAPACITY, ERR_TIMEOUT, ERR_OS = range(6)
I32, I64 = 0, 1


class ShmtError(RuntimeError):
    """A libshmt call returned a non-zero status."""

    def __init__(self, code: int, text: str):
        super().__init__(text)
        self.code = code


class NpyInfo(C.Structure):
    _fields_ = [
        ("descr", C.c_char * 8),
        ("ndim", C.c_int32),
        ("fortran_order", C.c_int32),
        ("shape", C.c_int64 * 8),
        ("data_offset", C.c_int64),
        ("file_size", C.c_int64),
        ("ptr", C.c_int64),
        ("fd", C.c_int64),
    ]


_vp, _i, _i64, _u64, _d, _s = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_double, C.c_char_p
_pvp, _pi64 = C.POINTER(C.c_void_p), C.POINTER(C.c_int64)

# name -> (restype, argtypes); must list every function include/shmt.h declares
SIGNATURES = {
    "shmt_last_error": (_s, []),
    "shmt_version": (_i, []),
    "shmt_ctx_create": (_i, [_i, _pvp]),
    "shmt_ctx_destroy": (_i, [_vp]),
    "shmt_ctx_scratch_bytes": (_i64, [_vp]),
    "shmt_ctx_check": (_i, [_vp, _vp]),
    "shmt_ctx_reserve": (_i, [_vp, _i64, _i64, _vp]),
    "shmt_ctx_reserve_minibatch": (_i, [_vp, _i64, _pi64, _i, _vp]),
    "shmt_map_table_bytes": (_i64, [_i64, _i64]),
    "shmt_map_create": (_i, [_i, _i64, _i64, _i, _i, _vp, _vp, _pvp]),
    "shmt_map_insert": (_i, [_vp, _vp, _vp, _i64, _vp]),
    "shmt_map_erase": (_i, [_vp, _vp, _i64, _vp, _vp]),
    "shmt_map_query": (_i, [_vp, _vp, _i, _i64, _vp, _vp]),
    "shmt_map_capacity": (_i64, [_vp]),
    "shmt_map_memory_usage": (_i64, [_vp]),
    "shmt_map_size": (_i64, [_vp]),
    "shmt_map_key_dtype": (_i, [_vp]),
    "shmt_map_val_dtype": (_i, [_vp]),
    "shmt_map_destroy": (_i, [_vp]),
    "shmt_fetch": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i64, _i64, _vp, _vp]),
    "shmt_device_fault": (_i, [C.POINTER(C.c_int)]),
    "shmt_fetch_partitioned": (_i, [_vp, _pvp, _i, _i, _vp, _vp, _i, _i64, _i64, _vp, _vp]),
    "shmt_set": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i64, _i64, _vp, _vp]),
    "shmt_insert_set": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i64, _i64, _vp, _vp]),
    "shmt_scan": (_i, [_vp, _vp, _i, _i64, _i, _vp]),
    "shmt_scan_static": (_i, [_vp, _i, _i64, _i, _vp]),
    "shmt_scan_static_check": (_i, [_vp]),
    "shmt_debug_lookback_timeout": (_i, [_vp, _vp]),
    "shmt_relabel": (_i, [_vp, _pvp, _pi64, _i, _i, _vp, _vp, _pi64, _vp]),
    "shmt_sample_hop": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i, _u64,
                             _u64, _vp, _vp, _pi64, _vp]),
    "shmt_sample_hop_eids": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i, _u64,
                                  _u64, _vp, _vp, _vp, _pi64, _vp]),
    "shmt_sample_hop_weighted": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i,
                                      _u64, _u64, _vp, _vp, _vp, _pi64, _vp]),
    "shmt_subcsr_edge_base": (_i, [_vp, _i, _vp, _i, _i64, _vp, _vp]),
    "shmt_sample_minibatch": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i64, _pi64, _i, _i, _u64,
                                   _u64, _pvp, _pvp, _pvp, _pvp, _pi64, _vp]),
    "shmt_sample_minibatch_weighted": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _pi64, _i, _i,
                                            _u64, _u64, _pvp, _pvp, _pvp, _pvp, _pi64, _vp]),
    "shmt_sample_minibatch_eids": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i64, _pi64, _i, _i, _u64,
                                        _u64, _pvp, _pvp, _pvp, _pvp, _pvp, _pi64, _vp]),
    "shmt_subcsr_count": (_i, [_vp, _vp, _i, _vp, _i, _i64, _vp, _pi64, _vp]),
    "shmt_subcsr_fill": (_i, [_vp, _i, _vp, _i, _vp, _i, _i64, _vp, _vp, _vp]),
    "shmt_shm_create": (_i, [_s, _i64, _i, _pi64, _pi64]),
    "shmt_shm_open": (_i, [_s, _i64, _i, _pi64, _pi64]),
    "shmt_shm_create_excl": (_i, [_s, _i64, _i, _pi64, _pi64]),
    "shmt_shm_unlink": (_i, [_s]),
    "shmt_shm_release": (_i, [_s, _i64, _i64, _i64, _i]),
    "shmt_shm_exists": (_i, [_s]),
    "shmt_npy_open": (_i, [_s, _i, C.POINTER(NpyInfo)]),
    "shmt_npy_close": (_i, [_i64, _i64, _i64, _i]),
    "shmt_host_register": (_i, [_vp, _i64]),
    "shmt_host_unregister": (_i, [_vp]),
    "shmt_host_prefault": (_i, [_vp, _i64, _i]),
    "shmt_host_numa_nodes": (_i, []),
    "shmt_host_numa_place": (_i, [_vp, _i64, _i, _i]),
    "shmt_dev_alloc": (_i, [_i64, _pvp]),
    "shmt_dev_free": (_i, [_vp]),
    "shmt_ipc_get_handle": (_i, [_vp, _vp]),
    "shmt_ipc_open_handle": (_i, [_vp, _pvp]),
    "shmt_ipc_close_handle": (_i, [_vp]),
    "shmt_stream_read": (_i, [_vp, _i64, _vp, _vp]),
    "shmt_random_read": (_i, [_vp, _i64, _i64, _i, _u64, _vp, _vp]),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m shmtensor_b200.build` (needs nvcc). There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    return lib.shmt_last_error().decode(errors="replace")


def check(rc: int) -> None:
    """Raise :class:`ShmtError` carrying the library's message if ``rc`` is non-zero."""
    if rc != OK:
        raise ShmtError(rc, last_error())
