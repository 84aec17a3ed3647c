"""Seeded random sweep: shapes, transpose modes, paddings, scalars and kernel ids drawn at
random (fixed seeds, so every run sees the same cases), each compared with the oracle
and checked for writes outside C.  Complements the hand-picked edge cases."""
import numpy as np
import pytest

from helpers import Case, run_and_check

pytestmark = pytest.mark.gpu



def _draw(rng, dtype, table_size):
    # extents: mostly small/ragged, sometimes a few tiles wide; log-uniform-ish
    def extent(hi):
        return int(min(hi, max(1, round(np.exp(rng.uniform(0.0, np.log(hi)))))))
    m, n, k = extent(700), extent(700), extent(900)
    ta, tb = bool(rng.integers(2)), bool(rng.integers(2))
    align = {"f16": 8, "f32": 4, "f64": 1}[dtype]
    mode = rng.integers(3)
    if mode == 0:
        pad = (0, 0, 0)
    elif mode == 1:  # arbitrary padding (unaligned leading dimensions)
        pad = tuple(int(x) for x in rng.integers(0, 9, 3))
    else:            # padding that makes every leading dimension a multiple of the vector width
        from helpers import lead_dims
        pad = tuple(int((-x) % align + align * rng.integers(0, 3)) for x in lead_dims(ta, tb, m, n, k))
    alpha = float(rng.choice([1.0, -1.0, 0.5, 1.75]))
    beta = float(rng.choice([0.0, 1.0, -0.25, 0.5]))
    kid = int(rng.integers(-1, table_size))  # -1 = automatic, else any row of the table
    return ta, tb, m, n, k, alpha, beta, pad, kid


@pytest.mark.parametrize("dtype,seed,count", [("f16", 101, 60), ("f32", 202, 60), ("f64", 303, 30)])
def test_random_cases(cuda, mm, oracle, dtype, seed, count):
    rng = np.random.default_rng(seed)
    table_size = mm.num_kernels(dtype)
    for i in range(count):
        ta, tb, m, n, k, alpha, beta, pad, kid = _draw(rng, dtype, table_size)
        case = Case(oracle, dtype, ta, tb, m, n, k, alpha, beta, pad=pad, seed=seed * 1000 + i,
                    dist=oracle.DIST_NORMAL, scale=0.5, c_poison=(beta == 0.0))
        try:
            run_and_check(cuda, mm, case, kid)
        except AssertionError as e:
            raise AssertionError(f"case {i}: {dtype} ta={ta} tb={tb} m={m} n={n} k={k} alpha={alpha} beta={beta} "
                                 f"pad={pad} kernel={kid}: {e}") from e
