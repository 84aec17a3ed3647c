"""Build recipe for libmmbo_gemm.so and the C++ harness (nvcc, sm_100a only).

The library is built in-tree (gemm_mmbo_b200/_build/) so that the built file travels with
a snapshot of the repository to a GPU machine.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import pathlib
import shutil
import subprocess

PKG = pathlib.Path(__file__).resolve().parent
ROOT = PKG.parent
BUILD = PKG / "_build"
LIB = BUILD / "libmmbo_gemm.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-ffp-contract=off",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(exe).exists():
        raise RuntimeError("nvcc not found; libmmbo_gemm.so cannot be built")
    return exe


def _newer(target: pathlib.Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(pathlib.Path(s).stat().st_mtime <= t for s in sources)


def library_sources() -> list[pathlib.Path]:
    return sorted((PKG / "csrc").glob("*.cu*")) + sorted((PKG / "csrc").glob("*.h")) + \
        sorted((ROOT / "include").glob("*.h*"))


def build_library(force: bool = False, verbose: bool = False) -> pathlib.Path:
    srcs = library_sources()
    if not force and _newer(LIB, srcs):
        return LIB
    BUILD.mkdir(exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", str(LIB), str(PKG / "csrc" / "mmbo_api.cu"), "-lcudart"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return LIB


def build_harness(force: bool = False) -> list[pathlib.Path]:
    """C++ benchmark / test programs (the counterparts of the reference's
    src/gemm/benchmark.cc and src/gemm/test.cc), linked against the library."""
    build_library(force=False)
    out = []
    for name in ("benchmark", "test_gemm"):
        src = PKG / "harness" / f"{name}.cc"
        if not src.exists():
            continue
        exe = BUILD / name
        if not force and _newer(exe, [src, LIB, *sorted((ROOT / "include").glob("*.h*"))]):
            out.append(exe)
            continue
        cmd = [_nvcc(), "-x", "cu", *NVCC_FLAGS, "-I", str(ROOT / "include"),
               "-o", str(exe), str(src), f"-L{BUILD}", "-lmmbo_gemm", "-lcudart", "-lcublas",
               "-Xlinker", "-rpath=$ORIGIN"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {name}:\n{res.stdout}\n{res.stderr}")
        out.append(exe)
    return out


if __name__ == "__main__":
    import sys
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_harness(force="--force" in sys.argv))
