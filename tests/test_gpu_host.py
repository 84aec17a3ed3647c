"""GEMM on host-resident operands (mmbo_gemm_f16_host / mmbo_gemm_f32_host / mmbo_gemm_f64_host): the library
stages A once and pipelines column panels of B and C; results must equal the oracle's
within the dtype's tolerance and host padding rows must stay untouched."""
import numpy as np
import pytest

from helpers import Case, TOL, bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["f16", "f32", "f64"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_host_operands_match_oracle(cuda, mm, oracle, dtype, ta, tb):
    # n spans several 256-column panels (ragged last one); m and k ragged as well
    for (m, n, k, beta) in [(300, 2600, 200, 0.5), (129, 515, 77, 0.0), (64, 100, 0, 0.5)]:
        case = Case(oracle, dtype, ta, tb, m, n, k, 1.25, beta, pad=(8, 16, 24) if dtype == "f16" else (3, 5, 7),
                    dist=oracle.DIST_NORMAL, scale=0.5, c_poison=(beta == 0.0))
        C = case.C.copy()
        mm.gemm_host(dtype, ta, tb, m, n, k, 1.25, case.A, case.lda, case.B, case.ldb, beta, C, case.ldc)
        assert mm.device_status() == 0
        assert np.array_equal(bits(C[:, m:]), bits(case.C[:, m:])), "host padding rows written"
        err = oracle.rel_frobenius(dtype, m, n, np.ascontiguousarray(C), case.ldc, case.reference())
        assert err <= TOL[dtype], (m, n, k, err)


def test_host_operands_pinned_large(cuda, mm, oracle):
    """Pinned buffers, enough panels to wrap the two device buffers several times."""
    torch = cuda
    m, n, k = 1024, 8192, 512
    A = torch.from_numpy(oracle.fill("f16", m, k, mat=0, dist=1, scale=0.5)).pin_memory()
    B = torch.from_numpy(oracle.fill("f16", n, k, mat=1, dist=1, scale=0.5)).pin_memory()
    C = torch.from_numpy(oracle.fill("f16", m, n, mat=2, dist=1, scale=0.5)).pin_memory()
    C0 = C.clone()
    mm.gemm_host("f16", False, True, m, n, k, 1.0, A, m, B, n, 0.5, C, m)
    ref = oracle.gemm("f16", False, True, m, n, k, 1.0, A.numpy(), m, B.numpy(), n, 0.5, C0.numpy(), m)
    err = oracle.rel_frobenius("f16", m, n, C.numpy(), m, ref)
    assert err <= TOL["f16"], err
