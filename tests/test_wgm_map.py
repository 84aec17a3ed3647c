"""The tile remap: oracle and library (through the C ABI, host only) against the
reference's golden vector src/gemm/ref/res (fixture tests/golden/wgm_map_460x64_wgm8.npz,
made by tests/golden/make_wgm_golden.py) and, where it was compiled, against the
reference's own checker src/gemm/ref/map.cpp (oracle/_ref/map_ref)."""
import pathlib
import re
import subprocess

import numpy as np
import pytest

GOLD = pathlib.Path(__file__).parent / "golden" / "wgm_map_460x64_wgm8.npz"
REF_BIN = pathlib.Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "map_ref"


@pytest.fixture(scope="module")
def gold():
    g = np.load(GOLD)
    return g["pairs"].astype(np.uint32), int(g["nwg0"]), int(g["nwg1"]), int(g["wgm"])


def test_golden_is_complete(gold):
    pairs, nwg0, nwg1, wgm = gold
    assert (nwg0, nwg1, wgm) == (460, 64, 8) and pairs.shape == (460 * 64, 4)
    # file order: wg0 fastest
    assert np.array_equal(pairs[:, 0], np.tile(np.arange(460), 64))
    assert np.array_equal(pairs[:, 1], np.repeat(np.arange(64), 460))


def test_oracle_matches_golden(oracle, gold):
    pairs, nwg0, nwg1, wgm = gold
    grid = oracle.wgm_map_grid(nwg0, nwg1, wgm)
    assert np.array_equal(grid[pairs[:, 1], pairs[:, 0]], pairs[:, 2:4])


def test_library_matches_golden(mm, gold):
    pairs, nwg0, nwg1, wgm = gold
    got = np.array([mm.wgm_map(int(a), int(b), nwg0, nwg1, wgm) for a, b in pairs[:, :2]], dtype=np.uint32)
    assert np.array_equal(got, pairs[:, 2:4])


@pytest.mark.parametrize("nwg0,nwg1,wgm", [(460, 64, 8), (32, 64, 8), (7, 13, 8), (5, 3, 8), (64, 61, 16),
                                           (1, 1, 8), (9, 9, 1), (3, 100, 4)])
def test_map_is_a_bijection_and_library_equals_oracle(oracle, mm, nwg0, nwg1, wgm):
    grid = oracle.wgm_map_grid(nwg0, nwg1, wgm)
    flat = grid.reshape(-1, 2)
    assert flat[:, 0].max() < nwg0 and flat[:, 1].max() < nwg1
    assert len({(int(a), int(b)) for a, b in flat}) == nwg0 * nwg1
    for j in range(nwg1):
        for i in range(nwg0):
            t = tuple(int(x) for x in grid[j, i])
            assert mm.wgm_map(i, j, nwg0, nwg1, wgm) == t
            assert oracle.wgm_unmap(t[0], t[1], nwg0, nwg1, wgm) == (i, j)


def test_partial_last_block_rule(oracle):
    """Remainder-width rule of src/gemm/ref/Kernels.cpp:211-236: in the last, narrower
    block the divisor is nwg1 % wgm."""
    nwg0, nwg1, wgm = 10, 11, 8  # last block is 3 wide
    grid = oracle.wgm_map_grid(nwg0, nwg1, wgm)
    for j in range(8, 11):
        for i in range(nwg0):
            serial = i + (j % 8) * nwg0
            assert tuple(grid[j, i]) == (serial // 3, serial % 3 + 8)


@pytest.mark.skipif(not REF_BIN.exists(), reason="reference checker not compiled (no reference tree)")
def test_oracle_matches_reference_binary(oracle):
    out = subprocess.run([str(REF_BIN)], capture_output=True, check=True).stdout
    pat = re.compile(rb"\((\d+),(\d+)\)--->\s*\((\d+),\s*(\d+)\) in original map")
    rows = np.array([[int(g) for g in m.groups()] for m in pat.finditer(out)], dtype=np.uint32)
    assert rows.shape == (460 * 64, 4)
    grid = oracle.wgm_map_grid(460, 64, 8)
    assert np.array_equal(grid[rows[:, 1], rows[:, 0]], rows[:, 2:4])
    assert b"error" not in out  # the checker's own inverse test found nothing
