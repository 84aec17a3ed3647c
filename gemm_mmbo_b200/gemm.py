"""Python mirror of the reference's launch surface (src/gemm/gemm.h:4-5,47-48).

`gemm()` takes the reference's argument list -- (m, n, k, alpha, A, lda, B, ldb, beta, C,
ldc, kernelId) -- preceded by dtype and the two transpose flags; `sgemm_NT`, `hgemm_NT`,
... are the per-layout wrappers named after the reference's `dgemm_NT`.  A, B and C are
device buffers: torch CUDA tensors or raw device addresses.  Every call goes through
the C ABI; errors come back as `MmboError` carrying the library's status code (the
reference prints and exits: src/gemm/common.h:20-24).
"""
from __future__ import annotations

import ctypes

from ._lib import LIB

DTYPE_F32, DTYPE_F16, DTYPE_F64 = 0, 1, 2
KERNEL_AUTO = -1
DIST_UNIFORM, DIST_NORMAL, DIST_ZERO = 0, 1, 2
MAT_A, MAT_B, MAT_C = 0, 1, 2

_DTYPES = {"f32": DTYPE_F32, "f16": DTYPE_F16, "f64": DTYPE_F64, DTYPE_F32: DTYPE_F32, DTYPE_F16: DTYPE_F16,
           DTYPE_F64: DTYPE_F64}


class MmboError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: status {status}: {status_string(status)}")


def status_string(status: int) -> str:
    s = LIB.mmbo_status_string(int(status))
    return s.decode() if s else "?"


def _addr(x) -> int | None:
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return int(x.data_ptr())  # torch tensor


def _stream(stream) -> int | None:
    if stream is None:
        try:
            import torch
            if torch.cuda.is_available():
                return int(torch.cuda.current_stream().cuda_stream) or None
        except ImportError:
            pass
        return None
    if isinstance(stream, int):
        return stream or None
    return int(stream.cuda_stream) or None


def gemm(dtype, transA: bool, transB: bool, m: int, n: int, k: int, alpha: float, A, lda: int, B,
         ldb: int, beta: float, C, ldc: int, kernelId: int = KERNEL_AUTO, stream=None) -> None:
    """C = alpha*op(A)*op(B) + beta*C on the current device, asynchronously on `stream`
    (default: torch's current stream)."""
    dt = _DTYPES[dtype]
    name = {DTYPE_F32: "mmbo_gemm_f32", DTYPE_F16: "mmbo_gemm_f16", DTYPE_F64: "mmbo_gemm_f64"}[dt]
    scalar = ctypes.c_double if dt == DTYPE_F64 else ctypes.c_float
    a, b = scalar(alpha), scalar(beta)
    rc = getattr(LIB, name)(int(bool(transA)), int(bool(transB)), m, n, k, ctypes.byref(a), _addr(A), lda,
                            _addr(B), ldb, ctypes.byref(b), _addr(C), ldc, kernelId, _stream(stream))
    if rc != 0:
        raise MmboError(rc, name)


def gemm_bcast(transA: bool, transB: bool, m: int, n: int, k: int, alpha: float, A, lda: int, B, ldb: int,
               beta: float, C, ldc: int, peers, kernelId: int = KERNEL_AUTO, stream=None) -> None:
    """fp16 GEMM whose epilogue also stores the result to further copies of the C window
    (`peers`: addresses or tensors, e.g. the same window in other GPUs' memory)."""
    a, b = ctypes.c_float(alpha), ctypes.c_float(beta)
    arr = (ctypes.c_void_p * max(1, len(peers)))(*[_addr(p) for p in peers])
    rc = LIB.mmbo_gemm_f16_bcast(int(bool(transA)), int(bool(transB)), m, n, k, ctypes.byref(a), _addr(A), lda,
                                 _addr(B), ldb, ctypes.byref(b), _addr(C), ldc, arr, len(peers), kernelId,
                                 _stream(stream))
    if rc != 0:
        raise MmboError(rc, "mmbo_gemm_f16_bcast")


def gemm_mcast(transA: bool, transB: bool, m: int, n: int, k: int, alpha: float, A, lda: int, B, ldb: int,
               beta: float, C, ldc: int, C_multicast, kernelId: int = KERNEL_AUTO, stream=None) -> None:
    """fp16 GEMM whose epilogue writes the result once to `C_multicast`, a multicast address of the C
    window (NVSwitch delivers every store to all GPUs bound to it); old C is read from `C`."""
    a, b = ctypes.c_float(alpha), ctypes.c_float(beta)
    rc = LIB.mmbo_gemm_f16_mcast(int(bool(transA)), int(bool(transB)), m, n, k, ctypes.byref(a), _addr(A), lda,
                                 _addr(B), ldb, ctypes.byref(b), _addr(C), ldc, _addr(C_multicast), kernelId,
                                 _stream(stream))
    if rc != 0:
        raise MmboError(rc, "mmbo_gemm_f16_mcast")


def gemm_sharded(n_gpus: int, rank: int, nccl_comm: int | None, gather_c: bool, transA: bool, transB: bool, m: int,
                 n: int, k: int, alpha: float, A, lda: int, B_block, ldb: int, beta: float, C, ldc: int,
                 kernelId: int = KERNEL_AUTO, stream=None) -> None:
    """This rank's part of an fp16 GEMM sharded by column blocks (mmbo_gemm_f16_sharded): C is the whole
    m x n matrix on this GPU, B_block this rank's block of op(B); with gather_c the blocks are exchanged
    over NCCL (`nccl_comm`: address of the ncclComm_t) so that every rank ends with all of C."""
    a, b = ctypes.c_float(alpha), ctypes.c_float(beta)
    rc = LIB.mmbo_gemm_f16_sharded(n_gpus, rank, nccl_comm, int(bool(gather_c)), int(bool(transA)), int(bool(transB)),
                                   m, n, k, ctypes.byref(a), _addr(A), lda, _addr(B_block), ldb, ctypes.byref(b),
                                   _addr(C), ldc, kernelId, _stream(stream))
    if rc != 0:
        raise MmboError(rc, "mmbo_gemm_f16_sharded")


def gemm_sharded_host(n_gpus: int, rank: int, nccl_comm: int | None, transA: bool, transB: bool, m: int, n: int,
                      k: int, alpha: float, A, lda: int, B_block, ldb: int, beta: float, C_block, ldc: int,
                      kernelId: int = KERNEL_AUTO) -> None:
    """The same on host operands (mmbo_gemm_f16_sharded_host): each rank uploads its share of A, the shares
    are exchanged between the GPUs over NVLink; B_block / C_block are this rank's column blocks."""
    a, b = ctypes.c_float(alpha), ctypes.c_float(beta)
    rc = LIB.mmbo_gemm_f16_sharded_host(n_gpus, rank, nccl_comm, int(bool(transA)), int(bool(transB)), m, n, k,
                                        ctypes.byref(a), _haddr(A), lda, _haddr(B_block), ldb, ctypes.byref(b),
                                        _haddr(C_block), ldc, kernelId)
    if rc != 0:
        raise MmboError(rc, "mmbo_gemm_f16_sharded_host")


def gemm_host(dtype, transA: bool, transB: bool, m: int, n: int, k: int, alpha: float, A, lda: int, B,
              ldb: int, beta: float, C, ldc: int, kernelId: int = KERNEL_AUTO) -> None:
    """Same GEMM with A, B, C in host memory (pinned torch tensors, numpy arrays or raw
    addresses); returns when C holds the result."""
    dt = _DTYPES[dtype]
    name = {DTYPE_F32: "mmbo_gemm_f32_host", DTYPE_F16: "mmbo_gemm_f16_host", DTYPE_F64: "mmbo_gemm_f64_host"}[dt]
    scalar = ctypes.c_double if dt == DTYPE_F64 else ctypes.c_float
    a, b = scalar(alpha), scalar(beta)
    rc = getattr(LIB, name)(int(bool(transA)), int(bool(transB)), m, n, k, ctypes.byref(a), _haddr(A), lda,
                            _haddr(B), ldb, ctypes.byref(b), _haddr(C), ldc, kernelId)
    if rc != 0:
        raise MmboError(rc, name)


def _haddr(x):
    if x is None or isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    return int(x.ctypes.data)  # numpy


def gemm_strided_batched(dtype, transA, transB, m, n, k, alpha, A, lda, strideA, B, ldb, strideB, beta, C, ldc,
                         strideC, batch, kernelId: int = KERNEL_AUTO, stream=None) -> None:
    """`batch` independent GEMMs whose operands are `stride*` elements apart."""
    dt = _DTYPES[dtype]
    scalar = ctypes.c_double if dt == DTYPE_F64 else ctypes.c_float
    a, b = scalar(alpha), scalar(beta)
    rc = LIB.mmbo_gemm_strided_batched(dt, int(bool(transA)), int(bool(transB)), m, n, k,
                                       ctypes.cast(ctypes.byref(a), ctypes.c_void_p), _addr(A), lda, strideA,
                                       _addr(B), ldb, strideB, ctypes.cast(ctypes.byref(b), ctypes.c_void_p),
                                       _addr(C), ldc, strideC, batch, kernelId, _stream(stream))
    if rc != 0:
        raise MmboError(rc, "mmbo_gemm_strided_batched")


def _wrap(dtype, ta, tb):
    def f(m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId=KERNEL_AUTO, stream=None):
        gemm(dtype, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kernelId, stream)
    f.__doc__ = (f"{dict(f32='s', f16='h', f64='d')[dtype]}gemm_{'T' if ta else 'N'}{'T' if tb else 'N'}: "
                 "argument order of the reference's dgemm_NT (src/gemm/gemm.h:47-48).")
    return f


sgemm_NN, sgemm_NT = _wrap("f32", False, False), _wrap("f32", False, True)
sgemm_TN, sgemm_TT = _wrap("f32", True, False), _wrap("f32", True, True)
hgemm_NN, hgemm_NT = _wrap("f16", False, False), _wrap("f16", False, True)
hgemm_TN, hgemm_TT = _wrap("f16", True, False), _wrap("f16", True, True)
dgemm_NN, dgemm_NT = _wrap("f64", False, False), _wrap("f64", False, True)
dgemm_TN, dgemm_TT = _wrap("f64", True, False), _wrap("f64", True, True)


def num_kernels(dtype) -> int:
    return int(LIB.mmbo_num_kernels(_DTYPES[dtype]))


def kernel_name(dtype, kernel_id: int) -> str:
    s = LIB.mmbo_kernel_name(_DTYPES[dtype], kernel_id)
    if s is None:
        raise MmboError(-7, "mmbo_kernel_name")
    return s.decode()


def kernel_params(dtype, kernel_id: int) -> dict:
    out = (ctypes.c_int * 8)()
    rc = LIB.mmbo_kernel_params(_DTYPES[dtype], kernel_id, out)
    if rc != 0:
        raise MmboError(rc, "mmbo_kernel_params")
    keys = ("MT0", "MT1", "threads", "DepthU", "stages", "ctaGroup", "wgm", "tensorCores")
    return dict(zip(keys, list(out)))


def kernel_table(dtype) -> list[dict]:
    """The counterpart of the tables in src/gemm/constants.h:4-135."""
    return [{"id": i, "name": kernel_name(dtype, i), **kernel_params(dtype, i)}
            for i in range(num_kernels(dtype))]


def select_kernel(dtype, transA, transB, m, n, k, A, lda, B, ldb, C, ldc) -> int:
    rc = LIB.mmbo_select_kernel(_DTYPES[dtype], int(bool(transA)), int(bool(transB)), m, n, k, _addr(A), lda,
                                _addr(B), ldb, _addr(C), ldc)
    if rc < 0:
        raise MmboError(rc, "mmbo_select_kernel")
    return rc


def wgm_map(wg0: int, wg1: int, nwg0: int, nwg1: int, wgm: int) -> tuple[int, int]:
    a, b = ctypes.c_uint32(), ctypes.c_uint32()
    LIB.mmbo_wgm_map(wg0, wg1, nwg0, nwg1, wgm, ctypes.byref(a), ctypes.byref(b))
    return a.value, b.value


def shard_columns(n: int, n_gpus: int, rank: int, align: int = 128) -> tuple[int, int]:
    """(first column, number of columns) of B/C owned by `rank`."""
    c0, nc = ctypes.c_size_t(), ctypes.c_size_t()
    rc = LIB.mmbo_shard_columns(n, n_gpus, rank, align, ctypes.byref(c0), ctypes.byref(nc))
    if rc != 0:
        raise MmboError(rc, "mmbo_shard_columns")
    return c0.value, nc.value


def fill(dtype, dst, rows: int, cols: int, ld: int, *, seed: int = 1234, mat: int = 0, dist: int = 0,
         scale: float = 1.0, row0: int = 0, col0: int = 0, total_rows: int | None = None,
         stream=None) -> None:
    """Seeded operand generation on the device (include/mmbo_rng.h)."""
    dt = _DTYPES[dtype]
    fn = {DTYPE_F32: LIB.mmbo_fill_f32, DTYPE_F16: LIB.mmbo_fill_f16, DTYPE_F64: LIB.mmbo_fill_f64}[dt]
    rc = fn(_addr(dst), rows, cols, ld, seed, mat, dist, float(scale), row0, col0,
            rows if total_rows is None else total_rows, _stream(stream))
    if rc != 0:
        raise MmboError(rc, "mmbo_fill")


def device_status() -> int:
    """Synchronise the device; return its fault word (0 = none) and clear it."""
    v = ctypes.c_uint32()
    rc = LIB.mmbo_device_status(ctypes.byref(v))
    if rc > 0:
        raise MmboError(rc, "mmbo_device_status")
    return v.value


def workspace_bytes(dtype, kernel_id: int, m: int, n: int, k: int) -> int:
    """Scratch bytes a call with this kernel id needs (0: the kernel uses none)."""
    out = ctypes.c_size_t()
    rc = LIB.mmbo_gemm_workspace_bytes(_DTYPES[dtype], kernel_id, m, n, k, ctypes.byref(out))
    if rc != 0:
        raise MmboError(rc, "mmbo_gemm_workspace_bytes")
    return out.value


def set_workspace(buf, nbytes: int = 0) -> None:
    """Lend the library a device buffer (tensor or address) as scratch for the current
    device; `None` returns to library-managed scratch."""
    rc = LIB.mmbo_set_workspace(_addr(buf), nbytes)
    if rc != 0:
        raise MmboError(rc, "mmbo_set_workspace")


def tuning_set(dtype, transA: bool, transB: bool, m: int, n: int, k: int, kernel_id: int, split: int = 0) -> None:
    """Pin the kernel (and, optionally, how the contraction is split: 0 per call, 1 never, 2 always)
    automatic selection uses for one exact problem."""
    rc = LIB.mmbo_tuning_set_split(_DTYPES[dtype], int(bool(transA)), int(bool(transB)), m, n, k, kernel_id, split)
    if rc != 0:
        raise MmboError(rc, "mmbo_tuning_set_split")


def tuning_load(path) -> None:
    rc = LIB.mmbo_tuning_load(str(path).encode())
    if rc != 0:
        raise MmboError(rc, "mmbo_tuning_load")


def tuning_clear() -> None:
    LIB.mmbo_tuning_clear()


def set_option(name: str, value: int) -> None:
    """Set one of the library's experiment / diagnosis switches (see mmbo_set_option)."""
    rc = LIB.mmbo_set_option(name.encode(), int(value))
    if rc != 0:
        raise MmboError(rc, "mmbo_set_option")


def get_option(name: str) -> int:
    v = ctypes.c_uint32()
    rc = LIB.mmbo_get_option(name.encode(), ctypes.byref(v))
    if rc != 0:
        raise MmboError(rc, "mmbo_get_option")
    return v.value


def launch_count() -> int:
    """Kernel launches the library has queued since it was loaded."""
    return int(LIB.mmbo_launch_count())


def last_kernel(dtype) -> int:
    """Table row the most recent GEMM call of `dtype` ran (-1 before the first)."""
    return int(LIB.mmbo_last_kernel(_DTYPES[dtype]))
