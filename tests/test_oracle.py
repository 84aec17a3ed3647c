"""CPU checks of the oracle itself: the blocked GEMM against the literal triple loop
(bit equality) and against numpy, the generator's statistics and determinism, and the
binary16 conversions against numpy."""
import numpy as np
import pytest


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_blocked_equals_naive_and_numpy(oracle, dtype, ta, tb):
    O = oracle
    m, n, k = 37, 29, 53
    ra, rb = (k if ta else m), (n if tb else k)
    ca, cb = (m if ta else k), (k if tb else n)
    A = O.fill(dtype, ra, ca, ra + 3, mat=O.MAT_A)
    B = O.fill(dtype, rb, cb, rb + 3, mat=O.MAT_B)
    C = O.fill(dtype, m, n, m + 3, mat=O.MAT_C)
    fast = O.gemm(dtype, ta, tb, m, n, k, 1.5, A, ra + 3, B, rb + 3, -0.25, C, m + 3)
    slow = O.gemm(dtype, ta, tb, m, n, k, 1.5, A, ra + 3, B, rb + 3, -0.25, C, m + 3, naive=True)
    assert np.array_equal(fast, slow)
    a = A[:, :ra].astype(np.float64).T
    b = B[:, :rb].astype(np.float64).T
    opa = a.T if ta else a
    opb = b.T if tb else b
    want = 1.5 * (opa @ opb) - 0.25 * C[:, :m].astype(np.float64).T
    assert np.abs(fast.T - want).max() < 1e-12


def test_beta_zero_ignores_c(oracle):
    O = oracle
    A = O.fill("f32", 8, 8, mat=0)
    B = O.fill("f32", 8, 8, mat=1)
    C = np.full((8, 8), np.nan, dtype=np.float32)
    out = O.gemm("f32", False, False, 8, 8, 8, 2.0, A, 8, B, 8, 0.0, C, 8)
    assert np.isfinite(out).all()


def test_k_zero(oracle):
    O = oracle
    C = O.fill("f32", 5, 4, 7, mat=2)
    out = O.gemm("f32", False, True, 5, 4, 0, 3.0, None, 5, None, 4, 0.5, C, 7)
    assert np.array_equal(out.T, 0.5 * C[:, :5].astype(np.float64).T)


def test_fill_independent_of_ld_and_shard(oracle):
    O = oracle
    full = O.fill("f16", 40, 24, 40, seed=7, mat=O.MAT_B, dist=O.DIST_NORMAL, scale=0.5)
    padded = O.fill("f16", 40, 24, 51, seed=7, mat=O.MAT_B, dist=O.DIST_NORMAL, scale=0.5)
    assert np.array_equal(full.view(np.uint16), padded[:, :40].view(np.uint16))
    assert np.isnan(padded[:, 40:]).all()
    shard = O.fill("f16", 40, 8, 40, seed=7, mat=O.MAT_B, dist=O.DIST_NORMAL, scale=0.5, col0=8,
                   total_rows=40)
    assert np.array_equal(shard.view(np.uint16), full[8:16].view(np.uint16))


def test_fill_statistics(oracle):
    O = oracle
    u = O.fill("f32", 512, 512, dist=O.DIST_UNIFORM).astype(np.float64)
    assert -1.0 <= u.min() and u.max() < 1.0
    assert abs(u.mean()) < 5e-3 and abs(u.var() - 1.0 / 3.0) < 5e-3
    g = O.fill("f32", 512, 512, dist=O.DIST_NORMAL, scale=0.5).astype(np.float64)
    assert abs(g.mean()) < 5e-3 and abs(g.std() - 0.5) < 5e-3
    # fourth moment of a normal: 3 sigma^4
    assert abs((g ** 4).mean() / 0.5 ** 4 - 3.0) < 0.1


def test_fill_known_answers(oracle):
    """Pins the generator: first elements for seed 1234 (values produced by this
    implementation; a change of generator must be deliberate)."""
    O = oracle
    u = O.fill("f32", 4, 1, seed=1234, mat=O.MAT_A, dist=O.DIST_UNIFORM)[0]
    g = O.fill("f32", 4, 1, seed=1234, mat=O.MAT_A, dist=O.DIST_NORMAL)[0]
    import json
    import pathlib
    gold = json.loads((pathlib.Path(__file__).parent / "golden" / "rng_known_answers.json").read_text())
    assert [int(x) for x in u.view(np.uint32)] == gold["uniform_seed1234_matA_bits"]
    assert [int(x) for x in g.view(np.uint32)] == gold["normal_seed1234_matA_bits"]


def test_half_conversion_matches_numpy(oracle):
    O = oracle
    # every finite binary16 value survives fill -> float16 via numpy comparison
    x = O.fill("f32", 4096, 16, dist=O.DIST_NORMAL, scale=3.0)
    h = O.fill("f16", 4096, 16, dist=O.DIST_NORMAL, scale=3.0)
    assert np.array_equal(x.astype(np.float16).view(np.uint16), h.view(np.uint16))
    tiny = O.fill("f32", 4096, 16, dist=O.DIST_NORMAL, scale=1e-6)
    tiny_h = O.fill("f16", 4096, 16, dist=O.DIST_NORMAL, scale=1e-6)
    assert np.array_equal(tiny.astype(np.float16).view(np.uint16), tiny_h.view(np.uint16))


def test_rel_frobenius(oracle):
    O = oracle
    ref = np.arange(12, dtype=np.float64).reshape(3, 4) + 1.0
    got = ref.astype(np.float32)
    assert O.rel_frobenius("f32", 4, 3, got, 4, ref) == 0.0
    got[1, 2] += 1.0
    want = 1.0 / np.sqrt((ref ** 2).sum())
    assert abs(O.rel_frobenius("f32", 4, 3, got, 4, ref) - want) < 1e-12
    got[0, 0] = np.nan
    assert np.isnan(O.rel_frobenius("f32", 4, 3, got, 4, ref))


def test_sampled_matches_full(oracle):
    O = oracle
    m, n, k = 33, 21, 40
    A = O.fill("f16", k, m, k + 8, mat=0)
    B = O.fill("f16", k, n, k + 8, mat=1)
    C = O.fill("f16", m, n, m, mat=2)
    full = O.gemm("f16", True, False, m, n, k, 0.75, A, k + 8, B, k + 8, 0.5, C, m)
    rows = np.array([0, 5, 32, 17]); cols = np.array([0, 20, 3, 9])
    s = O.gemm_sampled("f16", True, False, k, 0.75, A, k + 8, B, k + 8, 0.5, C, m, rows, cols)
    assert np.array_equal(s, full[cols, rows])
