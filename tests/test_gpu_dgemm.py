"""DGEMM (binary64, the reference's own data type) against the oracle's long-double
accumulation: relative Frobenius error <= 1e-13, all transpose modes, ragged shapes,
padded leading dimensions, the reference's HPL update (alpha = -1, beta = 1, NT)."""
import pytest

from helpers import Case, run_and_check

pytestmark = pytest.mark.gpu

MODES = [(False, False), (False, True), (True, False), (True, True)]
SHAPES = [(1, 1, 1), (5, 3, 2), (64, 64, 16), (65, 63, 17), (129, 127, 33), (200, 300, 100), (257, 130, 129)]


@pytest.mark.parametrize("kernel_id", [0, 1, 2, 3, 4, -1])
@pytest.mark.parametrize("ta,tb", MODES)
def test_dgemm_shapes(cuda, mm, oracle, kernel_id, ta, tb):
    for (m, n, k) in SHAPES:
        for pad in ((0, 0, 0), (3, 1, 2)):
            case = Case(oracle, "f64", ta, tb, m, n, k, -1.0, 1.0, pad=pad, seed=m + 31 * n)
            run_and_check(cuda, mm, case, kernel_id)


@pytest.mark.parametrize("kernel_id", [0, 1, 2, 3, 4])
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


@pytest.mark.parametrize("ta,tb", MODES)
def test_dgemm_persistent_kernel_many_tiles(cuda, mm, oracle, ta, tb):
    """More tiles than resident CTAs (each CTA walks several), ragged edges in m and n, a K tail
    that is not a multiple of the slab depth; even leading dimensions (bulk-copy rows where the
    operand's tile rows are contiguous) and odd ones (element copies everywhere)."""
    m, n, k = 128 * 22 + 10, 64 * 15 + 6, 100
    for pad in ((0, 0, 0), (1, 1, 3)):
        case = Case(oracle, "f64", ta, tb, m, n, k, -1.0, 1.0, pad=pad, seed=77)
        ref = case.reference()
        for kid in (3, 4):
            run_and_check(cuda, mm, case, kid, ref=ref)


def test_dgemm_misaligned_base_pointers(cuda, mm, oracle):
    """Operands that start 8 bytes off a 16-byte boundary: bulk copies cannot address them, the
    producer warps fall back to element copies."""
    import numpy as np
    torch = cuda
    m, n, k = 300, 200, 70
    case = Case(oracle, "f64", False, True, m, n, k, -1.0, 1.0, pad=(2, 2, 2))
    devs = []
    for host in (case.A, case.B, case.C):
        buf = torch.zeros(host.size + 3, dtype=torch.float64, device="cuda")
        off = 1 if buf.data_ptr() % 16 == 0 else 2
        buf[off:off + host.size].copy_(torch.from_numpy(host.reshape(-1)))
        devs.append((buf, off))
    dA, dB, dC = (b[o:o + h.size] for (b, o), h in zip(devs, (case.A, case.B, case.C)))
    assert dA.data_ptr() % 16 == 8 and dB.data_ptr() % 16 == 8
    for kid in (2, 3, 4):
        dC.copy_(torch.from_numpy(case.C.reshape(-1)))
        mm.gemm("f64", False, True, m, n, k, -1.0, dA, case.lda, dB, case.ldb, 1.0, dC, case.ldc, kid)
        torch.cuda.synchronize()
        assert mm.device_status() == 0
        got = dC.cpu().numpy().reshape(case.C.shape)
        assert np.array_equal(got[:, m:].view(np.uint64), case.C[:, m:].view(np.uint64))
        err = oracle.rel_frobenius("f64", m, n, np.ascontiguousarray(got), case.ldc, case.reference())
        assert err <= 1e-13, (kid, err)


def test_dgemm_kernels_agree_on_a_larger_problem(cuda, mm, oracle):
    """1536 x 1024 x 512 (too slow for the long-double oracle at full size to be worth it in every
    mode): the tensor kernels must agree with the one-thread-per-element kernel to rounding."""
    import numpy as np
    torch = cuda
    m, n, k = 1536, 1024, 512
    A = torch.empty(k * m, dtype=torch.float64, device="cuda")
    B = torch.empty(k * n, dtype=torch.float64, device="cuda")
    mm.fill("f64", A, m, k, m, mat=0)
    mm.fill("f64", B, n, k, n, mat=1)
    outs = {}
    for kid in (0, 2, 3, 4):
        C = torch.empty(n * m, dtype=torch.float64, device="cuda")
        mm.fill("f64", C, m, n, m, mat=2)
        mm.gemm("f64", False, True, m, n, k, -1.0, A, m, B, n, 1.0, C, m, kid)
        torch.cuda.synchronize()
        assert mm.device_status() == 0
        outs[kid] = C.cpu().numpy()
    scale = np.linalg.norm(outs[0])
    for kid in (2, 3, 4):
        assert np.linalg.norm(outs[kid] - outs[0]) / scale <= 1e-14, kid


@pytest.mark.parametrize("ta,tb", MODES)
def test_dgemm_operand_feed_paths(cuda, mm, oracle, ta, tb):
    """Each operand either goes through its tensor map (even leading dimension) or through
    element copies (odd): all four combinations, both tile heights, ragged edges and a K tail."""
    m, n, k = 330, 202, 90
    for pad_a in (0, 1):
        for pad_b in (0, 1):
            case = Case(oracle, "f64", ta, tb, m, n, k, 1.5, -0.5, pad=(pad_a, pad_b, 1), seed=5 + 2 * pad_a + pad_b)
            ref = case.reference()
            for kid in (3, 4):
                run_and_check(cuda, mm, case, kid, ref=ref)
