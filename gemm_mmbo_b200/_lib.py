"""ctypes binding of libmmbo_gemm.so (declarations: include/mmbo_gemm.h).

There is no fallback of any kind: if the CUDA library has not been built, importing
this module raises.  Build it with `python -m gemm_mmbo_b200.build`.
"""
from __future__ import annotations

import ctypes
import pathlib

_PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = _PKG / "_build" / "libmmbo_gemm.so"

_sz = ctypes.c_size_t
_vp = ctypes.c_void_p
_fp = ctypes.POINTER(ctypes.c_float)
_dp = ctypes.POINTER(ctypes.c_double)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_szp = ctypes.POINTER(ctypes.c_size_t)

# name -> (restype, argtypes); every symbol declared in include/mmbo_gemm.h
SIGNATURES = {
    "mmbo_gemm_f32": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz,
                                     _fp, _vp, _sz, ctypes.c_int, _vp]),
    "mmbo_gemm_f16": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz,
                                     _fp, _vp, _sz, ctypes.c_int, _vp]),
    "mmbo_gemm_f16_bcast": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz,
                                           _fp, _vp, _sz, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                           ctypes.c_int, _vp]),
    "mmbo_gemm_f16_mcast": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz,
                                           _fp, _vp, _sz, _vp, ctypes.c_int, _vp]),
    "mmbo_gemm_f16_sharded": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                             _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz, _fp, _vp, _sz, ctypes.c_int, _vp]),
    "mmbo_gemm_f16_sharded_host": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int, ctypes.c_int, _sz, _sz,
                                                  _sz, _fp, _vp, _sz, _vp, _sz, _fp, _vp, _sz, ctypes.c_int]),
    "mmbo_gemm_f64": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _dp, _vp, _sz, _vp, _sz,
                                     _dp, _vp, _sz, ctypes.c_int, _vp]),
    "mmbo_fill_f64": (ctypes.c_int, [_vp, _sz, _sz, _sz, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int,
                                     ctypes.c_float, _sz, _sz, _sz, _vp]),
    "mmbo_gemm_f32_host": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz,
                                          _fp, _vp, _sz, ctypes.c_int]),
    "mmbo_gemm_f16_host": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz,
                                          _fp, _vp, _sz, ctypes.c_int]),
    "mmbo_gemm_f64_host": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _dp, _vp, _sz, _vp, _sz,
                                          _dp, _vp, _sz, ctypes.c_int]),
    "mmbo_gemm_strided_batched": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _vp, _vp,
                                                 _sz, _sz, _vp, _sz, _sz, _vp, _vp, _sz, _sz, _sz, ctypes.c_int, _vp]),
    "mmbo_num_kernels": (ctypes.c_int, [ctypes.c_int]),
    "mmbo_kernel_name": (ctypes.c_char_p, [ctypes.c_int, ctypes.c_int]),
    "mmbo_kernel_params": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]),
    "mmbo_select_kernel": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _vp, _sz,
                                          _vp, _sz, _vp, _sz]),
    "mmbo_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "mmbo_tuning_set": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, ctypes.c_int]),
    "mmbo_tuning_set_split": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, ctypes.c_int,
                                             ctypes.c_int]),
    "mmbo_tuning_load": (ctypes.c_int, [ctypes.c_char_p]),
    "mmbo_tuning_clear": (None, []),
    "mmbo_wgm_map": (None, [ctypes.c_uint32] * 5 + [_u32p, _u32p]),
    "mmbo_shard_columns": (ctypes.c_int, [_sz, ctypes.c_int, ctypes.c_int, _sz, _szp, _szp]),
    "mmbo_fill_f32": (ctypes.c_int, [_vp, _sz, _sz, _sz, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int,
                                     ctypes.c_float, _sz, _sz, _sz, _vp]),
    "mmbo_fill_f16": (ctypes.c_int, [_vp, _sz, _sz, _sz, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int,
                                     ctypes.c_float, _sz, _sz, _sz, _vp]),
    "mmbo_device_status": (ctypes.c_int, [_u32p]),
    "mmbo_debug_trace": (ctypes.c_int, [ctypes.c_int, _vp, _sz]),
    "mmbo_selftest_bounded_wait": (ctypes.c_int, [ctypes.c_ulonglong, _vp]),
    "mmbo_gemm_workspace_bytes": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _szp]),
    "mmbo_set_workspace": (ctypes.c_int, [_vp, _sz]),
    "mmbo_set_option": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_uint]),
    "mmbo_get_option": (ctypes.c_int, [ctypes.c_char_p, _u32p]),
    "mmbo_launch_count": (ctypes.c_ulonglong, []),
    "mmbo_last_kernel": (ctypes.c_int, [ctypes.c_int]),
    "mmbo_gemm_f32_noalloc": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, _fp, _vp, _sz, _vp, _sz,
                                             _fp, _vp, _sz, _vp]),
}


def load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m gemm_mmbo_b200.build`). There is no CPU fallback.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


LIB = load()

# The packaged tuning table (written by gemm_mmbo_b200.autotune on a B200) is loaded once;
# MMBO_TUNING_FILE, when set, is read by the library itself and takes its place.
import os as _os  # noqa: E402
_TABLE = _PKG / "tuning" / "b200.tbl"
if _TABLE.exists() and not _os.environ.get("MMBO_TUNING_FILE") and not _os.environ.get("MMBO_NO_TUNING"):
    LIB.mmbo_tuning_load(str(_TABLE).encode())
