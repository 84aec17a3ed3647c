"""gemm_mmbo_b200 -- host-side mirror of the GEMM launch surface over libmmbo_gemm.so.

The library itself is CUDA C++ (gemm_mmbo_b200/csrc, C ABI in include/mmbo_gemm.h); this
package only binds it for Python callers (tests, benchmark, multi-GPU driver).
"""
from .gemm import (  # noqa: F401
    DTYPE_F16, DTYPE_F32, KERNEL_AUTO, MmboError, device_status, fill, gemm, hgemm_NN, hgemm_NT,
    hgemm_TN, hgemm_TT, kernel_name, kernel_params, kernel_table, num_kernels, select_kernel,
    sgemm_NN, sgemm_NT, sgemm_TN, sgemm_TT, shard_columns, status_string, wgm_map,
)
