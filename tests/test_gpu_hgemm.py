"""HGEMM parity (fp16 storage, fp32 accumulation): every fp16 kernel of the table and
automatic selection against the oracle, relative Frobenius error <= 2e-3."""
import numpy as np
import pytest

from helpers import Case, run_and_check

pytestmark = pytest.mark.gpu

MODES = [(False, False), (False, True), (True, False), (True, True)]
# 0/1/several/partial tiles of the 256x128 and 128x128 macro-tiles; K tails of the
# 64-deep stage; more tiles than stages and than accumulators; odd numbers of
# 128-column blocks so that a CTA pair's second half falls outside C
SHAPES = [(8, 8, 8), (64, 32, 16), (128, 128, 64), (256, 128, 128), (136, 72, 200), (264, 136, 72),
          (520, 392, 328), (1024, 512, 640), (40, 1000, 96), (1000, 40, 96)]


@pytest.mark.parametrize("kernel_id", [1, 2, 3, 4, 5, 6, 7, -1, 0])
@pytest.mark.parametrize("ta,tb", MODES)
def test_hgemm_shapes(cuda, mm, oracle, kernel_id, ta, tb):
    for (m, n, k) in SHAPES:
        for pad, beta in (((0, 0, 0), 0.5), ((8, 16, 24), -0.25), ((0, 8, 0), 0.0)):
            case = Case(oracle, "f16", ta, tb, m, n, k, 1.0 if beta else 0.75, beta, pad=pad,
                        seed=m * 7 + n, dist=oracle.DIST_NORMAL, scale=0.5)
            run_and_check(cuda, mm, case, kernel_id)


@pytest.mark.parametrize("kernel_id", [1, 2, 3, 4, 5, 6, 7, -1, 0])
def test_hgemm_beta_zero_never_reads_c(cuda, mm, oracle, kernel_id):
    case = Case(oracle, "f16", False, True, 264, 200, 72, 2.0, 0.0, pad=(0, 8, 16), c_poison=True)
    run_and_check(cuda, mm, case, kernel_id)


@pytest.mark.parametrize("kernel_id", [1, 2, 3, 4, 5, 6, 7, -1])
def test_hgemm_many_tiles_per_cta(cuda, mm, oracle, kernel_id):
    """More tiles than SMs: every persistent CTA walks several tiles, so stage and
    accumulator phases wrap many times."""
    case = Case(oracle, "f16", False, True, 4096 + 8, 2048 + 8, 136, 1.0, 0.5, dist=oracle.DIST_NORMAL,
                scale=0.5)
    run_and_check(cuda, mm, case, kernel_id)


@pytest.mark.parametrize("kernel_id", [4, 5])
@pytest.mark.parametrize("beta", [0.0, 1.0])
def test_hgemm_short_contraction_rows_walk_many_tiles(cuda, mm, oracle, kernel_id, beta):
    """The rows built for short contractions (two epilogue warps per tensor-memory quarter; old C requested a
    tile ahead into a second set of staging buffers, or five operand stages with an L2 prefetch of the next
    tile's C): six or more tiles per CTA pair, so that every staging buffer, accumulator and barrier phase
    wraps several times, with and without old C, in two layouts."""
    for ta, tb, (m, n, k) in ((False, True, (256 * 40, 256 * 12, 136)), (True, False, (256 * 21 + 64, 256 * 22 + 32, 200))):
        case = Case(oracle, "f16", ta, tb, m, n, k, -1.0, beta, dist=oracle.DIST_NORMAL, scale=0.5,
                    c_poison=(beta == 0.0), seed=kernel_id)
        run_and_check(cuda, mm, case, kernel_id)


def test_hgemm_unaligned_operands(cuda, mm, oracle):
    """Leading dimensions that are not multiples of 8 cannot be described to TMA: small
    problems take the general kernel, large ones (and forced tensor-core rows) are realigned
    through scratch and run on the tensor cores; results are the same either way."""
    from helpers import to_device
    small = Case(oracle, "f16", False, True, 100, 60, 50, 1.0, 0.5, pad=(3, 3, 3))
    _, dA = to_device(cuda, small.A)
    _, dB = to_device(cuda, small.B)
    _, dC = to_device(cuda, small.C)
    assert mm.select_kernel("f16", False, True, 100, 60, 50, dA, small.lda, dB, small.ldb, dC, small.ldc) == 0
    for kid in (-1, 1, 2, 3, 4):
        run_and_check(cuda, mm, small, kid)
    for ta, tb in MODES:
        big = Case(oracle, "f16", ta, tb, 515, 389, 301, 1.0, 0.5, pad=(1, 3, 5), dist=oracle.DIST_NORMAL, scale=0.5)
        _, dA = to_device(cuda, big.A)
        _, dB = to_device(cuda, big.B)
        _, dC = to_device(cuda, big.C)
        assert mm.select_kernel("f16", ta, tb, 515, 389, 301, dA, big.lda, dB, big.ldb, dC, big.ldc) != 0
        for kid in (-1, 3, 4):
            run_and_check(cuda, mm, big, kid)


def test_hgemm_misaligned_base_pointers(cuda, mm, oracle):
    """A, B, C that start 2 bytes off a 16-byte boundary (sub-matrix views into a larger
    allocation) under otherwise TMA-friendly leading dimensions."""
    import numpy as np
    torch = cuda
    m, n, k = 520, 392, 328
    case = Case(oracle, "f16", False, True, m, n, k, 1.0, 0.5, pad=(8, 8, 8), dist=oracle.DIST_NORMAL, scale=0.5)
    devs = []
    for host in (case.A, case.B, case.C):
        buf = torch.zeros(host.size + 1, dtype=torch.float16, device="cuda")
        buf[1:].copy_(torch.from_numpy(host.reshape(-1)))
        devs.append(buf)
    dA, dB, dC = (b[1:] for b in devs)
    assert dA.data_ptr() % 16 == 2
    mm.gemm("f16", False, True, m, n, k, 1.0, dA, case.lda, dB, case.ldb, 0.5, dC, case.ldc, 3)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    got = dC.cpu().numpy().reshape(case.C.shape)
    assert np.array_equal(got[:, m:].view(np.uint16), case.C[:, m:].view(np.uint16))
    assert float(devs[2][0]) == 0.0  # the element before C untouched
    err = oracle.rel_frobenius("f16", m, n, np.ascontiguousarray(got), case.ldc, case.reference())
    assert err <= 2e-3, err


def test_hgemm_k_zero_and_empty(cuda, mm, oracle):
    run_and_check(cuda, mm, Case(oracle, "f16", False, False, 72, 40, 0, 2.0, 0.5, pad=(0, 0, 8)), -1)
    run_and_check(cuda, mm, Case(oracle, "f16", False, False, 0, 40, 16, 1.0, 0.5), -1)


def test_hgemm_tensor_kernels_agree_bitwise_across_runs(cuda, mm, oracle):
    from helpers import to_device
    torch = cuda
    case = Case(oracle, "f16", True, False, 520, 392, 328, 1.0, 0.5)
    outs = []
    for _ in range(2):
        _, dA = to_device(torch, case.A)
        _, dB = to_device(torch, case.B)
        _, dC = to_device(torch, case.C)
        mm.gemm("f16", True, False, 520, 392, 328, 1.0, dA, case.lda, dB, case.ldb, 0.5, dC, case.ldc, 1)
        torch.cuda.synchronize()
        outs.append(dC.cpu().numpy().view(np.uint16))
    assert np.array_equal(outs[0], outs[1])


def _pad_to8(ta, tb, m, n, k, extra=8):
    """Pads that make every leading dimension a multiple of 8 (TMA-addressable) while
    leaving `extra` or more padding rows below each matrix."""
    from helpers import lead_dims
    return tuple((-x) % 8 + extra for x in lead_dims(ta, tb, m, n, k))


@pytest.mark.parametrize("kernel_id", [1, 2, 3, 4, 5, 6, 7, -1])
@pytest.mark.parametrize("ta,tb", MODES)
def test_hgemm_ragged_extents_with_aligned_leading_dims(cuda, mm, oracle, kernel_id, ta, tb):
    """m, n, k that are not multiples of 8 under 8-aligned leading dimensions: the tensor
    core kernels run (TMA can address A and B) and must not touch the padding rows of C."""
    for (m, n, k) in [(100, 60, 50), (1001, 77, 130), (37, 129, 65), (257, 255, 7), (7, 9, 3)]:
        for beta in (0.5, 0.0):
            case = Case(oracle, "f16", ta, tb, m, n, k, 1.0, beta, pad=_pad_to8(ta, tb, m, n, k),
                        dist=oracle.DIST_NORMAL, scale=0.5, c_poison=(beta == 0.0))
            run_and_check(cuda, mm, case, kernel_id)


def test_hgemm_c_with_odd_leading_dim(cuda, mm, oracle):
    """Only A and B need TMA-friendly layouts; C may have any leading dimension."""
    m, n, k = 264, 136, 72
    case = Case(oracle, "f16", False, True, m, n, k, 1.0, 0.5, pad=(0, 0, 3), dist=oracle.DIST_NORMAL, scale=0.5)
    from helpers import to_device
    _, dA = to_device(cuda, case.A)
    _, dB = to_device(cuda, case.B)
    _, dC = to_device(cuda, case.C)
    assert mm.select_kernel("f16", False, True, m, n, k, dA, case.lda, dB, case.ldb, dC, case.ldc) != 0
    for kid in (1, 2, 3, 4, -1):
        run_and_check(cuda, mm, case, kid)


@pytest.mark.parametrize("kernel_id", [-1, 1, 2, 3, 4, 5, 6, 7])
def test_hgemm_result_stored_to_further_copies(cuda, mm, oracle, kernel_id):
    """mmbo_gemm_f16_bcast with the further copies on the same GPU: every copy must hold the same
    bits as C, rows below the matrix untouched; beta != 0 reads the old values from C only."""
    import numpy as np
    torch = cuda
    m, n, k = 520, 392, 328
    case = Case(oracle, "f16", False, True, m, n, k, 1.0, 0.5, pad=(0, 0, 8), dist=oracle.DIST_NORMAL, scale=0.5)
    dA = torch.from_numpy(case.A.reshape(-1)).cuda()
    dB = torch.from_numpy(case.B.reshape(-1)).cuda()
    dC = torch.from_numpy(case.C.reshape(-1)).cuda()
    copies = [torch.full((case.C.size,), 7.0, dtype=torch.float16, device="cuda") for _ in range(3)]
    mm.gemm_bcast(False, True, m, n, k, 1.0, dA, case.lda, dB, case.ldb, 0.5, dC, case.ldc, copies, kernel_id)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    got = dC.cpu().numpy().reshape(case.C.shape)
    err = oracle.rel_frobenius("f16", m, n, np.ascontiguousarray(got), case.ldc, case.reference())
    assert err <= 2e-3, err
    for c in copies:
        h = c.cpu().numpy().reshape(case.C.shape)
        assert np.array_equal(h[:, :m].view(np.uint16), got[:, :m].view(np.uint16))
        assert (h[:, m:] == 7.0).all(), "padding rows of a copy written"


def test_hgemm_bcast_refuses_what_tma_cannot_store(cuda, mm, oracle):
    torch = cuda
    m, n, k = 260, 128, 64  # m not a multiple of 8: the TMA epilogue would spill into padding rows
    A = torch.zeros(264 * k, dtype=torch.float16, device="cuda")
    B = torch.zeros(n * k, dtype=torch.float16, device="cuda")
    C = torch.zeros(n * 264, dtype=torch.float16, device="cuda")
    with pytest.raises(mm.MmboError) as e:
        mm.gemm_bcast(False, True, m, n, k, 1.0, A, 264, B, n, 0.0, C, 264, [C])
    assert e.value.status == -8  # MMBO_ERR_KERNEL_UNSUITABLE
    with pytest.raises(mm.MmboError):
        mm.gemm_bcast(False, True, 256, n, k, 1.0, A, 256, B, n, 0.0, C, 256, [C] * 8)  # more than 7 copies


@pytest.mark.gpu
def test_last_kernel_reports_the_row_an_automatic_call_ran(cuda, mm, oracle):
    """Automatic selection depends on beta (short contractions: the row that requests old C a tile ahead only pays
    when there is old C), which `select_kernel` cannot see; `last_kernel` names the row that actually ran."""
    import torch
    m = n = 4096
    k = 256
    A = (torch.randn((m, k), device="cuda") * 0.5).half()   # TN: A stored k x m, B stored k x n
    B = (torch.randn((n, k), device="cuda") * 0.5).half()
    C = torch.zeros((n, m), dtype=torch.float16, device="cuda")
    mm.gemm("f16", True, False, m, n, k, 1.0, A, k, B, k, 0.0, C, m)
    no_c = mm.last_kernel("f16")
    mm.gemm("f16", True, False, m, n, k, 1.0, A, k, B, k, 1.0, C, m)
    with_c = mm.last_kernel("f16")
    mm.gemm("f16", True, False, m, n, k, 1.0, A, k, B, k, 1.0, C, m, 3)
    forced = mm.last_kernel("f16")
    torch.cuda.synchronize()
    names = [mm.kernel_name("f16", i) for i in (no_c, with_c)]
    assert forced == 3
    assert "S5_CG2_WG320" in names[0] and "S3_CG2_WG320" in names[1], names


@pytest.mark.parametrize("kernel_id", [2, 3, 5, 6])
def test_hgemm_chain_on_one_stream_sees_the_previous_result(cuda, mm, oracle, kernel_id):
    """Back-to-back launches overlap their set-up with the end of the kernel before them (programmatic dependent
    launch): a GEMM whose operand is the C of the GEMM queued just before it on the same stream must still read the
    finished C.  Ten chained pairs, each compared bitwise with the same pair run with a synchronize in between and
    with the overlap switched off."""
    torch = cuda
    m = n = k = 512
    gen = torch.Generator(device="cuda").manual_seed(7 + kernel_id)
    A = (torch.randn((k, m), device="cuda", generator=gen) * 0.25).half()
    B = (torch.randn((n, k), device="cuda", generator=gen) * 0.25).half()
    B2 = (torch.randn((n, m), device="cuda", generator=gen) * 0.25).half()

    def pair(sync_between):
        C1 = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
        C2 = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
        mm.gemm("f16", False, False, m, n, k, 1.0, A, m, B, k, 0.0, C1, m, kernel_id)
        if sync_between:
            torch.cuda.synchronize()
        mm.gemm("f16", False, False, m, n, n, 1.0, C1, m, B2, n, 0.0, C2, m, kernel_id)  # op(A) of the second = C of the first
        torch.cuda.synchronize()
        return C2.cpu().numpy().view(np.uint16)

    before = mm.get_option("pdl")
    try:
        mm.set_option("pdl", 0)
        want = pair(True)
        mm.set_option("pdl", 1)
        assert np.isfinite(want.view(np.float16)).all()
        for _ in range(10):
            assert np.array_equal(pair(False), want)
    finally:
        mm.set_option("pdl", before)
