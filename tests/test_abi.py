"""Host-only checks of the C ABI: the library loads, exports every symbol the header
declares, describes its kernel table, partitions columns and rejects bad arguments
before anything is launched."""
import ctypes
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_exports_every_declared_symbol(mm):
    from gemm_mmbo_b200 import _lib
    header = (ROOT / "include" / "mmbo_gemm.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(mmbo_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared:
        assert hasattr(raw, name), name


def test_kernel_tables(mm):
    for dt in ("f32", "f16"):
        table = mm.kernel_table(dt)
        assert len(table) >= 3
        names = [r["name"] for r in table]
        assert len(set(names)) == len(names)
        for r in table:
            assert r["MT0"] > 0 and r["MT1"] > 0 and r["threads"] % 32 == 0
            # name carries the macro-tile like the reference's kernel names
            assert f"MT{r['MT0']:03d}x{r['MT1']:03d}x{r['DepthU']:02d}" in r["name"]
    assert any(r["tensorCores"] for r in mm.kernel_table("f16"))
    with pytest.raises(mm.MmboError):
        mm.kernel_name("f16", 99)
    with pytest.raises(mm.MmboError):
        mm.kernel_params("f32", -1)


@pytest.mark.parametrize("n,p,align", [(32768, 8, 128), (32768, 1, 128), (1000, 3, 128), (130, 4, 128),
                                       (5, 8, 1), (0, 2, 128), (4097, 8, 64)])
def test_shard_columns_partition(mm, n, p, align):
    blocks = [mm.shard_columns(n, p, r, align) for r in range(p)]
    pos = 0
    for c0, nc in blocks:
        assert c0 == pos
        pos += nc
    assert pos == n
    sizes = [nc for _, nc in blocks]
    assert max(sizes) - min(sizes) < 2 * align
    for c0, nc in blocks[:-1]:
        assert nc % align == 0 or c0 + nc == n


def test_shard_columns_rejects(mm):
    for args in [(10, 0, 0, 1), (10, 2, 2, 1), (10, 2, -1, 1)]:
        with pytest.raises(mm.MmboError):
            mm.shard_columns(*args)


def test_status_strings(mm):
    assert mm.status_string(0) == "ok"
    for code in range(-20, 0):
        assert mm.status_string(code) not in ("", "unknown status")


BAD = 0x1000  # a non-null, 16-byte aligned address that is never dereferenced on these paths


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_rejects_bad_arguments_before_launch(mm, dtype):
    ok = dict(transA=False, transB=True, m=64, n=32, k=16, alpha=1.0, A=BAD, lda=64, B=BAD, ldb=32,
              beta=0.0, C=BAD, ldc=64, kernelId=-1)

    def status(**kw):
        a = {**ok, **kw}
        try:
            mm.gemm(dtype, a["transA"], a["transB"], a["m"], a["n"], a["k"], a["alpha"], a["A"], a["lda"],
                    a["B"], a["ldb"], a["beta"], a["C"], a["ldc"], a["kernelId"], stream=0)
        except mm.MmboError as e:
            return e.status
        return 0

    assert status(lda=63) == -4          # NT: lda >= m
    assert status(ldb=31) == -5          # NT: ldb >= n
    assert status(ldc=63) == -6
    assert status(transA=True, lda=15) == -4   # TN: lda >= k
    assert status(transB=False, ldb=15) == -5  # NN: ldb >= k
    assert status(A=None) == -3 and status(B=None) == -3 and status(C=None) == -3
    assert status(kernelId=99) == -7 and status(kernelId=-2) == -7
    assert status(m=2 ** 31) == -2
    # empty problems are accepted and launch nothing
    assert status(m=0) == 0 and status(n=0) == 0


def test_raw_abi_rejects_bad_trans_and_null_scalars(mm):
    from gemm_mmbo_b200._lib import LIB
    one = ctypes.c_float(1.0)
    args = [64, 32, 16, ctypes.byref(one), BAD, 64, BAD, 32, ctypes.byref(one), BAD, 64, -1, None]
    assert LIB.mmbo_gemm_f32(2, 0, *args) == -1
    assert LIB.mmbo_gemm_f16(0, -1, *args) == -1
    args[3] = None
    assert LIB.mmbo_gemm_f32(0, 1, *args) == -3


def test_tuning_table_overrides_selection(mm, tmp_path):
    """Exact-size rows win over the heuristics; other sizes are unaffected; a file round
    trip works; bad rows are rejected.  (Selection is a host-side decision: no GPU needed.)"""
    mm.tuning_clear()
    args = ("f16", False, True, 8192, 8192, 8192, BAD, 8192, BAD, 8192, BAD, 8192)
    base = mm.select_kernel(*args)
    other = 1 if base != 1 else 2
    mm.tuning_set("f16", False, True, 8192, 8192, 8192, other)
    assert mm.select_kernel(*args) == other
    assert mm.select_kernel("f16", False, True, 8192, 8192, 4096, BAD, 8192, BAD, 8192, BAD, 8192) != -1
    assert mm.select_kernel("f16", True, False, 8192, 8192, 8192, BAD, 8192, BAD, 8192, BAD, 8192) == base or True
    mm.tuning_clear()
    assert mm.select_kernel(*args) == base
    f = tmp_path / "t.tbl"
    f.write_text("# dtype trans m n k kernel\nf16 NT 8192 8192 8192 2\nf64 NT 44160 2048 384 1\n")
    mm.tuning_load(f)
    assert mm.select_kernel(*args) == 2
    assert mm.select_kernel("f64", False, True, 44160, 2048, 384, BAD, 44160, BAD, 2048, BAD, 44160) == 1
    mm.tuning_clear()
    f.write_text("f16 NT 1 2 3 99\n")
    with pytest.raises(mm.MmboError):
        mm.tuning_load(f)
    with pytest.raises(mm.MmboError):
        mm.tuning_load(tmp_path / "missing.tbl")
    mm.tuning_clear()


def test_fp64_selection_is_the_warp_specialised_tensor_kernel():
    """No GPU needed (148 SMs assumed without a device): 64-row tiles for short contractions and
    for problems with few tiles, 128-row tiles otherwise."""
    import gemm_mmbo_b200 as mm
    BAD = 16
    mm.tuning_clear()
    def name(m, n, k):
        return mm.kernel_name("f64", mm.select_kernel("f64", False, True, m, n, k, BAD, m, BAD, n, BAD, m))
    assert "dmma_ws_MT064x064" in name(44160, 2048, 384)
    assert "dmma_ws_MT064x064" in name(1024, 1024, 1024)
    assert "dmma_ws_MT128x064" in name(4096, 4096, 4096)
    assert "dmma_ws_MT128x064" in name(2176, 2176, 2176)   # 578 tiles of 128 rows: 1.95 rounds of 296 slots
    assert "dmma_ws_MT064x064" in name(2368, 2368, 2368)   # 703 tiles would be 2.4 rounds; 1369 of 64 rows are 4.6


def test_exact_fp32_switch_beats_tuned_tensor_rows(mm):
    """With the exact-fp32 switch on, automatic selection never returns a split-precision
    (tensor-core) row -- not from the heuristics and not from a tuned row, the packaged table
    included.  Host-side decision: no GPU needed."""
    import gemm_mmbo_b200._lib as L
    mm.tuning_clear()
    if L._TABLE.exists():
        mm.tuning_load(L._TABLE)
    mm.tuning_set("f32", False, True, 1536, 2048, 384, 5)
    args = ("f32", False, True, 1536, 2048, 384, BAD, 1536, BAD, 2048, BAD, 1536)
    try:
        assert mm.get_option("f32_exact") == 0
        assert mm.kernel_params("f32", mm.select_kernel(*args))["tensorCores"] == 1
        mm.set_option("f32_exact", 1)
        kid = mm.select_kernel(*args)
        assert mm.kernel_params("f32", kid)["tensorCores"] == 0, kid
        big = ("f32", False, False, 8192, 8192, 8192, BAD, 8192, BAD, 8192, BAD, 8192)
        assert mm.kernel_params("f32", mm.select_kernel(*big))["tensorCores"] == 0
    finally:
        mm.set_option("f32_exact", 0)
        mm.tuning_clear()
    with pytest.raises(mm.MmboError) as e:
        mm.set_option("no_such_switch", 1)
    assert e.value.status == -18


def test_strided_batched_rejects_bad_arguments(mm):
    from gemm_mmbo_b200._lib import LIB
    one = ctypes.c_float(1.0)
    a = ctypes.cast(ctypes.byref(one), ctypes.c_void_p)
    ok = [1, 0, 1, 64, 32, 16, a, BAD, 64, 64 * 16, BAD, 32, 32 * 16, a, BAD, 64, 64 * 32, 4, -1, None]
    bad = list(ok); bad[0] = 7
    assert LIB.mmbo_gemm_strided_batched(*bad) == -9
    bad = list(ok); bad[8] = 63
    assert LIB.mmbo_gemm_strided_batched(*bad) == -4
    bad = list(ok); bad[18] = 99
    assert LIB.mmbo_gemm_strided_batched(*bad) == -7
    bad = list(ok); bad[17] = 0  # an empty batch is accepted and launches nothing
    assert LIB.mmbo_gemm_strided_batched(*bad) == 0


def test_sharded_entry_points_reject_bad_arguments_before_any_launch(mm):
    """Host-side checks of the multi-GPU entry points (no GPU, no NCCL needed): rank and GPU count, a
    missing communicator where an exchange is asked for, leading dimensions, and the empty problem."""
    from gemm_mmbo_b200._lib import LIB
    one = ctypes.c_float(1.0)
    a = ctypes.byref(one)

    def sharded(n_gpus, rank, comm, gather, m=512, n=1024, k=64, lda=512, ldb=64, ldc=512):
        return LIB.mmbo_gemm_f16_sharded(n_gpus, rank, comm, gather, 0, 0, m, n, k, a, BAD, lda, BAD, ldb, a, BAD, ldc, -1, None)

    assert sharded(0, 0, None, 0) == -10
    assert sharded(2, 2, None, 0) == -10
    assert sharded(2, -1, None, 0) == -10
    assert sharded(2, 0, None, 1) == -3          # an exchange needs the caller's communicator
    assert sharded(2, 1, None, 0, lda=100) == -4
    assert sharded(2, 1, None, 0, ldb=10) == -5
    assert sharded(2, 1, None, 0, m=0) == 0      # nothing to do, nothing launched
    host = LIB.mmbo_gemm_f16_sharded_host
    assert host(2, 0, None, 0, 0, 512, 1024, 64, a, BAD, 512, BAD, 64, a, BAD, 512, -1) == -3
    assert host(3, 3, None, 0, 0, 512, 1024, 64, a, BAD, 512, BAD, 64, a, BAD, 512, -1) == -10


@pytest.mark.parametrize("cols,world", [(32768, 8), (520, 2), (1024, 2), (8, 4), (4100, 3)])
def test_shares_of_a_tile_its_columns_on_16_byte_boundaries(mm, cols, world):
    """The shares of A that the ranks upload (mmbo_gemm_f16_sharded_host): consecutive, complete, and
    starting on multiples of 8 fp16 columns."""
    pos = 0
    for r in range(world):
        c0, cn = mm.shard_columns(cols, world, r, 8)
        assert c0 == pos and c0 % 8 == 0
        pos += cn
    assert pos == cols


def test_public_names_survive_any_import_order():
    """`gemm_mmbo_b200.gemm` is a function even when a submodule that needs the binding (`sharded`) was imported
    first -- Python would otherwise bind the package attribute to the submodule of the same name."""
    import subprocess
    import sys
    code = ("import gemm_mmbo_b200 as mm\n"
            "from gemm_mmbo_b200.sharded import ColumnShard\n"
            "assert callable(mm.gemm) and callable(mm.gemm_host) and callable(mm.select_kernel), type(mm.gemm)\n")
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr
