"""gemm_mmbo_b200 -- host-side mirror of the GEMM launch surface over libmmbo_gemm.so.

The library itself is CUDA C++ (gemm_mmbo_b200/csrc, C ABI in include/mmbo_gemm.h); this
package only binds it for Python callers (tests, benchmark, multi-GPU driver).

The binding is loaded on first use of any public name, so that `gemm_mmbo_b200.build`
can be imported to (re)build the library.  There is no fallback: touching any GEMM
entry point without a built libmmbo_gemm.so raises ImportError.
"""
import importlib

_PUBLIC = (
    "DTYPE_F16", "DTYPE_F32", "DTYPE_F64", "dgemm_NN", "dgemm_NT", "dgemm_TN", "dgemm_TT", "KERNEL_AUTO", "DIST_UNIFORM", "DIST_NORMAL", "DIST_ZERO", "MAT_A", "MAT_B",
    "MAT_C", "MmboError", "device_status", "fill", "gemm", "gemm_bcast", "gemm_mcast", "gemm_sharded", "gemm_sharded_host", "gemm_host", "set_option", "get_option", "launch_count", "last_kernel", "gemm_strided_batched", "hgemm_NN", "hgemm_NT", "hgemm_TN", "hgemm_TT",
    "kernel_name", "kernel_params", "kernel_table", "num_kernels", "select_kernel", "sgemm_NN", "sgemm_NT",
    "sgemm_TN", "sgemm_TT", "shard_columns", "status_string", "wgm_map", "workspace_bytes", "set_workspace", "tuning_set", "tuning_load", "tuning_clear",
)
__all__ = list(_PUBLIC)


def _bind_public():
    """Bind the public names to the functions of the `gemm` submodule.  Importing that submodule makes Python set
    the package attribute `gemm` to the MODULE, which would hide the function of the same name; every internal
    importer of the submodule calls this afterwards, so `gemm_mmbo_b200.gemm(...)` works whatever was imported first."""
    mod = importlib.import_module(__name__ + ".gemm")  # loads libmmbo_gemm.so or raises
    for n in _PUBLIC:
        globals()[n] = getattr(mod, n)
    return mod


def __getattr__(name):
    if name in _PUBLIC:
        _bind_public()
        return globals()[name]
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
