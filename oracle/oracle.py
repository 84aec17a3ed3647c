"""ctypes loader for the CPU oracle (oracle/_build/liboracle.so).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the benchmark's
CPU-baseline leg; the product package never imports it.  The arithmetic it checks
against is documented in ref_gemm.c and wgm_map.c (with reference file:line citations).
"""
from __future__ import annotations

import ctypes
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "liboracle.so"
_lib = None

_sz = ctypes.c_size_t
_vp = ctypes.c_void_p


def build(force: bool = False) -> pathlib.Path:
    """Compile the oracle with the Makefile beside this file (gcc only)."""
    if force and _LIB_PATH.exists():
        _LIB_PATH.unlink()
    # make rebuilds only when a source is newer than the library
    try:
        subprocess.run(["make", "-C", str(_HERE), "all"], check=True, capture_output=True)
    except (OSError, subprocess.CalledProcessError):
        if not _LIB_PATH.exists():  # a prebuilt library is used as it is
            raise
    return _LIB_PATH


def build_ref(reference_root: str) -> pathlib.Path | None:
    """Compile the reference's own remap checker into oracle/_ref/ if its source exists."""
    src = pathlib.Path(reference_root) / "src/gemm/ref/map.cpp"
    if not src.exists():
        return None
    subprocess.run(["make", "-C", str(_HERE), "ref", f"REF={reference_root}"], check=True,
                   capture_output=True)
    return _HERE / "_ref" / "map_ref"


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        for name, half in (("oracle_gemm_f32", False), ("oracle_gemm_f16", True),
                           ("oracle_gemm_naive_f32", False), ("oracle_gemm_naive_f16", True)):
            f = getattr(L, name)
            f.restype = None
            f.argtypes = [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, ctypes.c_float, _vp, _sz,
                          _vp, _sz, ctypes.c_float, _vp, _sz, _vp, _sz]
        L.oracle_gemm_sampled.restype = None
        L.oracle_gemm_sampled.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, _sz,
                                          ctypes.c_float, _vp, _sz, _vp, _sz, ctypes.c_float,
                                          _vp, _sz, _sz, _vp, _vp, _vp]
        L.oracle_rel_frobenius.restype = ctypes.c_double
        L.oracle_rel_frobenius.argtypes = [ctypes.c_int, _sz, _sz, _vp, _sz, _vp, _sz]
        L.oracle_gemm_f64.restype = None
        L.oracle_gemm_f64.argtypes = [ctypes.c_int, ctypes.c_int, _sz, _sz, _sz, ctypes.c_double, _vp, _sz,
                                      _vp, _sz, ctypes.c_double, _vp, _sz, _vp, _sz]
        for name in ("oracle_fill_f32", "oracle_fill_f16", "oracle_fill_f64"):
            f = getattr(L, name)
            f.restype = None
            f.argtypes = [_vp, _sz, _sz, _sz, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int,
                          ctypes.c_float, _sz, _sz, _sz]
        L.oracle_num_threads.restype = ctypes.c_int
        L.oracle_set_num_threads.restype = None
        L.oracle_set_num_threads.argtypes = [ctypes.c_int]
        L.oracle_wgm_map_grid.restype = None
        L.oracle_wgm_map_grid.argtypes = [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, _vp]
        u32p = ctypes.POINTER(ctypes.c_uint32)
        for name in ("oracle_wgm_map", "oracle_wgm_unmap"):
            f = getattr(L, name)
            f.restype = None
            f.argtypes = [ctypes.c_uint32] * 5 + [u32p, u32p]
        _lib = L
    return _lib


DIST_UNIFORM, DIST_NORMAL, DIST_ZERO = 0, 1, 2
MAT_A, MAT_B, MAT_C = 0, 1, 2


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(_vp)


def _storage(dtype: str):
    return {"f32": np.float32, "f16": np.float16, "f64": np.float64}[dtype]


def fill(dtype: str, rows: int, cols: int, ld: int | None = None, *, seed: int = 1234,
         mat: int = 0, dist: int = DIST_UNIFORM, scale: float = 1.0, pad=np.nan,
         row0: int = 0, col0: int = 0, total_rows: int | None = None) -> np.ndarray:
    """Column-major (ld x cols) host array, returned as a numpy array of shape (cols, ld)
    so that element (i, j) is out[j, i].  Padding rows hold `pad` (NaN by default)."""
    ld = rows if ld is None else ld
    assert ld >= rows
    out = np.full((cols, ld), pad, dtype=_storage(dtype))
    fn = getattr(lib(), f"oracle_fill_{dtype}")
    fn(_ptr(out), rows, cols, ld, seed, mat, dist, float(scale), row0, col0,
       rows if total_rows is None else total_rows)
    return out


def gemm(dtype: str, transA: bool, transB: bool, m: int, n: int, k: int, alpha: float,
         A: np.ndarray, lda: int, B: np.ndarray, ldb: int, beta: float,
         C: np.ndarray | None, ldc: int, naive: bool = False) -> np.ndarray:
    """Unrounded binary64 result, shape (n, m) (column-major m x n, ld = m)."""
    out = np.empty((n, m), dtype=np.float64)
    if dtype == "f64":  # long-double accumulation; there is no separate naive variant
        naive = False
    name = f"oracle_gemm_{'naive_' if naive else ''}{dtype}"
    getattr(lib(), name)(int(transA), int(transB), m, n, k, float(alpha), _ptr(A), lda,
                         _ptr(B), ldb, float(beta), _ptr(C), ldc, _ptr(out), max(m, 1))
    return out


def gemm_sampled(dtype: str, transA: bool, transB: bool, k: int, alpha: float, A, lda, B, ldb,
                 beta: float, C, ldc, rows: np.ndarray, cols: np.ndarray) -> np.ndarray:
    rows = np.ascontiguousarray(rows, dtype=np.uintp)
    cols = np.ascontiguousarray(cols, dtype=np.uintp)
    out = np.empty(rows.shape[0], dtype=np.float64)
    lib().oracle_gemm_sampled(0 if dtype == "f32" else 1, int(transA), int(transB), k,
                              float(alpha), _ptr(A), lda, _ptr(B), ldb, float(beta), _ptr(C),
                              ldc, rows.shape[0], _ptr(rows), _ptr(cols), _ptr(out))
    return out


def rel_frobenius(dtype: str, m: int, n: int, got: np.ndarray, ldg: int,
                  ref: np.ndarray) -> float:
    """||got - ref||_F / ||ref||_F over the m x n window; got is (n, ldg) storage-typed."""
    return float(lib().oracle_rel_frobenius({"f32": 0, "f16": 1, "f64": 2}[dtype], m, n, _ptr(got), ldg,
                                            _ptr(ref), max(m, 1)))


def wgm_map_grid(nwg0: int, nwg1: int, wgm: int) -> np.ndarray:
    """Array [nwg1, nwg0, 2] with the remapped (wg0', wg1') of every work-group."""
    out = np.empty((nwg1, nwg0, 2), dtype=np.uint32)
    lib().oracle_wgm_map_grid(nwg0, nwg1, wgm, _ptr(out))
    return out


def wgm_unmap(m0: int, m1: int, nwg0: int, nwg1: int, wgm: int) -> tuple[int, int]:
    a, b = ctypes.c_uint32(), ctypes.c_uint32()
    lib().oracle_wgm_unmap(m0, m1, nwg0, nwg1, wgm, ctypes.byref(a), ctypes.byref(b))
    return a.value, b.value


def set_num_threads(n: int = 0) -> None:
    """n <= 0: one thread per host core, whatever OMP_NUM_THREADS says."""
    lib().oracle_set_num_threads(int(n))


def num_threads() -> int:
    return int(lib().oracle_num_threads())
