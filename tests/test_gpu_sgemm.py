"""SGEMM parity: every fp32 kernel of the table (and automatic selection) against the
oracle, relative Frobenius error <= 1e-5, all transpose modes, ragged shapes, padded
leading dimensions, guard bands, beta == 0 with poisoned C."""
import numpy as np
import pytest

from helpers import Case, run_and_check

pytestmark = pytest.mark.gpu

MODES = [(False, False), (False, True), (True, False), (True, True)]
# shapes chosen to give 0, 1, several and partial tiles in each dimension of the
# 128x128 and 64x64 macro-tiles, and K tails of the 16-deep slab
SHAPES = [(1, 1, 1), (5, 3, 2), (64, 64, 16), (65, 63, 17), (128, 128, 32), (129, 127, 33),
          (200, 300, 100), (384, 256, 64), (257, 513, 129)]


@pytest.mark.parametrize("kernel_id", [0, 1, 2, 3, 4, 5, 6, -1])
@pytest.mark.parametrize("ta,tb", MODES)
def test_sgemm_shapes(cuda, mm, oracle, kernel_id, ta, tb):
    for (m, n, k) in SHAPES:
        for pad in ((0, 0, 0), (3, 3, 3), (4, 8, 12)):
            case = Case(oracle, "f32", ta, tb, m, n, k, 1.5, -0.25, pad=pad, seed=m * 1000 + n)
            run_and_check(cuda, mm, case, kernel_id)


@pytest.mark.parametrize("kernel_id", [0, 1, 2, 3, 4, 5, 6, -1])
def test_sgemm_beta_zero_never_reads_c(cuda, mm, oracle, kernel_id):
    case = Case(oracle, "f32", False, True, 150, 70, 40, 2.0, 0.0, pad=(1, 2, 3), c_poison=True)
    run_and_check(cuda, mm, case, kernel_id)


@pytest.mark.parametrize("kernel_id", [0, 1, 2, 3, 4, 5, 6, -1])
def test_sgemm_k_zero_scales_c(cuda, mm, oracle, kernel_id):
    case = Case(oracle, "f32", False, False, 70, 33, 0, 2.0, 0.5, pad=(0, 0, 5))
    run_and_check(cuda, mm, case, kernel_id)
    case = Case(oracle, "f32", False, False, 70, 33, 0, 2.0, 0.0, pad=(0, 0, 5), c_poison=True)
    run_and_check(cuda, mm, case, kernel_id)


def test_sgemm_empty(cuda, mm, oracle):
    for (m, n) in ((0, 5), (5, 0), (0, 0)):
        case = Case(oracle, "f32", False, False, m, n, 7, 1.0, 1.0)
        run_and_check(cuda, mm, case, -1)


def test_sgemm_deterministic(cuda, mm, oracle):
    """Two runs of the same kernel give bit-identical C."""
    import numpy as np
    from helpers import to_device
    torch = cuda
    case = Case(oracle, "f32", True, False, 300, 260, 190, 1.0, 0.0)
    outs = []
    for _ in range(2):
        _, dA = to_device(torch, case.A)
        _, dB = to_device(torch, case.B)
        _, dC = to_device(torch, case.C)
        mm.gemm("f32", True, False, 300, 260, 190, 1.0, dA, case.lda, dB, case.ldb, 0.0, dC, case.ldc, 1)
        torch.cuda.synchronize()
        outs.append(dC.cpu().numpy().view(np.uint32))
    assert np.array_equal(outs[0], outs[1])


def test_sgemm_tf32x3_accuracy_large_k(cuda, mm, oracle):
    """The split-precision tensor-core kernels keep fp32-level accuracy over a long
    contraction (k = 8192): relative Frobenius error <= 1e-5, like the FFMA kernels."""
    case = Case(oracle, "f32", True, False, 384, 320, 8192, 1.0, 0.5)
    ref = case.reference()
    errs = {kid: run_and_check(cuda, mm, case, kid, ref=ref) for kid in (1, 3, 4, 5)}
    print("rel Frobenius:", errs)
    assert max(errs.values()) <= 1e-5


def test_sgemm_lent_workspace(cuda, mm, oracle):
    """With a caller-owned scratch buffer the library allocates nothing: a buffer of the
    advertised size works, a smaller one is refused before any launch."""
    torch = cuda
    m, n, k = 300, 200, 100
    need = mm.workspace_bytes("f32", 3, m, n, k)
    assert need > 0 and mm.workspace_bytes("f32", 1, m, n, k) == 0
    case = Case(oracle, "f32", False, True, m, n, k, 1.5, -0.25, pad=(3, 3, 3))
    buf = torch.empty(need + 1024, dtype=torch.uint8, device="cuda")
    base = (buf.data_ptr() + 1023) // 1024 * 1024
    try:
        mm.set_workspace(base, need)
        run_and_check(cuda, mm, case, 3)
        mm.set_workspace(base, need - 1024)
        with pytest.raises(mm.MmboError) as e:
            run_and_check(cuda, mm, case, 3)
        assert e.value.status == -15
        with pytest.raises(mm.MmboError):
            mm.set_workspace(base + 8, need)  # misaligned
    finally:
        mm.set_workspace(None)
    run_and_check(cuda, mm, case, 3)  # library-managed scratch again


def test_rejected_workspace_leaves_library_scratch_usable(cuda, mm, oracle):
    """A misaligned buffer is refused (-15) before any state changes: the library's own scratch is
    neither freed nor left dangling, and the next split-precision GEMM is still right."""
    case = Case(oracle, "f32", False, True, 300, 200, 100, 1.5, -0.25, pad=(3, 3, 3))
    ref = case.reference()
    mm.set_workspace(None)
    run_and_check(cuda, mm, case, 3, ref=ref)          # library-managed scratch now exists
    junk = cuda.empty(1 << 20, dtype=cuda.uint8, device="cuda")
    with pytest.raises(mm.MmboError) as e:
        mm.set_workspace(junk.data_ptr() // 1024 * 1024 + 1024 + 8, 1 << 19)
    assert e.value.status == -15
    run_and_check(cuda, mm, case, 3, ref=ref)
    run_and_check(cuda, mm, case, 5, ref=ref)


def test_lent_workspace_too_small_falls_back_on_automatic_selection(cuda, mm, oracle):
    """Automatic fp32 selection never fails for want of scratch: with a lent buffer that is too small
    for the split-precision rows it takes a CUDA-core kernel; a forced row still reports -15."""
    torch = cuda
    m = n = k = 640  # 640^3 > 512^3: automatic selection would take a split-precision row
    case = Case(oracle, "f32", False, False, m, n, k, 1.0, 0.0, c_poison=True)
    buf = torch.empty(4096 + 1024, dtype=torch.uint8, device="cuda")
    base = (buf.data_ptr() + 1023) // 1024 * 1024
    try:
        mm.set_workspace(base, 4096)
        run_and_check(cuda, mm, case, -1)
        with pytest.raises(mm.MmboError) as e:
            run_and_check(cuda, mm, case, 4)
        assert e.value.status == -15
    finally:
        mm.set_workspace(None)


def test_two_streams_share_the_library_scratch_safely(cuda, mm, oracle):
    """Default fp32 GEMMs (split-precision rows, which repack their operands into the one
    library-managed scratch buffer) queued on two streams with different operands: the library orders
    the scratch users on the GPU, so both results match the oracle."""
    torch = cuda
    cases = [Case(oracle, "f32", False, True, 768, 640, 700, 1.0, 0.5, seed=31),
             Case(oracle, "f32", True, False, 704, 832, 650, -1.0, 0.0, seed=32, c_poison=True)]
    refs = [c.reference() for c in cases]
    dev = [[torch.from_numpy(x).cuda() for x in (c.A, c.B, c.C)] for c in cases]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rep in range(4):  # several rounds, alternating streams, nothing in between
        for c, (dA, dB, dC), st in zip(cases, dev, streams):
            if rep:
                dC.copy_(torch.from_numpy(c.C), non_blocking=False)
            mm.gemm("f32", c.ta, c.tb, c.m, c.n, c.k, c.alpha, dA, c.lda, dB, c.ldb, c.beta, dC, c.ldc, -1, st)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    for c, (dA, dB, dC), ref in zip(cases, dev, refs):
        err = oracle.rel_frobenius("f32", c.m, c.n, np.ascontiguousarray(dC.cpu().numpy()), c.ldc, ref)
        assert err <= 1e-5, err


@pytest.mark.parametrize("ta,tb", MODES)
def test_sgemm_producer_consumer_ffma_kernel(cuda, mm, oracle, ta, tb):
    """fp32 id 6: more tiles than resident CTAs, ragged edges, a K tail; leading dimensions that
    allow TMA (multiples of 4, for the operands whose tile rows are contiguous) and ones that do not."""
    m, n, k = 128 * 20 + 12, 128 * 16 + 4, 100
    for pad in ((0, 0, 0), (1, 3, 2)):
        case = Case(oracle, "f32", ta, tb, m, n, k, 1.5, -0.25, pad=pad, seed=91)
        run_and_check(cuda, mm, case, 6)
