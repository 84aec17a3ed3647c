"""DGEMM (binary64, the reference's own data type) against the oracle's long-double
accumulation: relative Frobenius error <= 1e-13, all transpose modes, ragged shapes,
padded leading dimensions, the reference's HPL update (alpha = -1, beta = 1, NT)."""
import pytest

from helpers import Case, run_and_check

pytestmark = pytest.mark.gpu

MODES = [(False, False), (False, True), (True, False), (True, True)]
SHAPES = [(1, 1, 1), (5, 3, 2), (64, 64, 16), (65, 63, 17), (129, 127, 33), (200, 300, 100), (257, 130, 129)]


@pytest.mark.parametrize("kernel_id", [0, 1, 2, -1])
@pytest.mark.parametrize("ta,tb", MODES)
def test_dgemm_shapes(cuda, mm, oracle, kernel_id, ta, tb):
    for (m, n, k) in SHAPES:
        for pad in ((0, 0, 0), (3, 1, 2)):
            case = Case(oracle, "f64", ta, tb, m, n, k, -1.0, 1.0, pad=pad, seed=m + 31 * n)
            run_and_check(cuda, mm, case, kernel_id)


@pytest.mark.parametrize("kernel_id", [0, 1, 2])
def test_dgemm_beta_zero_and_k_zero(cuda, mm, oracle, kernel_id):
    run_and_check(cuda, mm, Case(oracle, "f64", False, True, 150, 70, 40, 2.0, 0.0, pad=(1, 2, 3), c_poison=True),
                  kernel_id)
    run_and_check(cuda, mm, Case(oracle, "f64", False, True, 70, 33, 0, 2.0, 0.5, pad=(0, 0, 5)), kernel_id)


def test_dgemm_reference_sweep_shape(cuda, mm, oracle):
    """One point of the reference's run.sh sweep (M multiple of 384, N = 2048, K = 384, ldc = 44160,
    alpha = -1, beta = 1, NT) through the reference-named Python mirror."""
    m, n, k = 1536, 2048, 384
    case = Case(oracle, "f64", False, True, m, n, k, -1.0, 1.0, pad=(0, 0, 44160 - m))
    run_and_check(cuda, mm, case, -1)


@pytest.mark.parametrize("dtype", ["f16", "f32", "f64"])
def test_strided_batched(cuda, mm, oracle, dtype):
    """Three problems packed back to back in one allocation each, through the batched entry."""
    import numpy as np
    from helpers import TOL
    torch = cuda
    m, n, k, batch = 136, 72, 200, 3
    cases = [Case(oracle, dtype, False, True, m, n, k, 1.0, 0.5, seed=100 + b) for b in range(batch)]
    tdt = {"f16": torch.float16, "f32": torch.float32, "f64": torch.float64}[dtype]
    dA = torch.from_numpy(np.stack([c.A for c in cases])).cuda()
    dB = torch.from_numpy(np.stack([c.B for c in cases])).cuda()
    dC = torch.from_numpy(np.stack([c.C for c in cases])).cuda()
    assert dA.dtype == tdt
    mm.gemm_strided_batched(dtype, False, True, m, n, k, 1.0, dA, m, m * k, dB, n, n * k, 0.5, dC, m, m * n, batch)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    out = dC.cpu().numpy()
    for b, case in enumerate(cases):
        err = oracle.rel_frobenius(dtype, m, n, np.ascontiguousarray(out[b]), m, case.reference())
        assert err <= TOL[dtype], (b, err)
