"""Strided-batched GEMM (mmbo_gemm_strided_batched): the counterpart of the batch index the
reference's general kernel takes from the third grid dimension (src/gemm/ref/Kernels.cpp:254,
strides src/gemm/gemm.h:62-69,88-92).  Every problem of a batch is compared with the oracle;
the call must cost one launch of the GEMM kernel wherever that kernel can address the batch."""
import numpy as np
import pytest

from helpers import Case, TOL, lead_dims, stored_cols

pytestmark = pytest.mark.gpu

MODES = [(False, False), (False, True), (True, False), (True, True)]
ALIGN = {"f16": 8, "f32": 4, "f64": 2}


def _batch(torch, mm, oracle, dtype, ta, tb, m, n, k, batch, alpha, beta, kid, pad_to=None, gap=0, seed=500):
    """Problems packed `stride` elements apart in one allocation per operand.  pad_to: leading
    dimensions and strides rounded up to this many elements (what TMA needs); gap: extra elements
    between problems."""
    ra, rb, rc = lead_dims(ta, tb, m, n, k)
    ca, cb, cc = stored_cols(ta, tb, m, n, k)
    up = (lambda x: x) if not pad_to else (lambda x: -(-x // pad_to) * pad_to)
    pads = (up(ra) - ra, up(rb) - rb, up(rc) - rc)
    cases = [Case(oracle, dtype, ta, tb, m, n, k, alpha, beta, pad=pads, seed=seed + b, dist=oracle.DIST_NORMAL,
                  scale=0.5, c_poison=(beta == 0.0)) for b in range(batch)]
    c0 = cases[0]
    sA, sB, sC = up(c0.lda * ca + gap), up(c0.ldb * cb + gap), up(c0.ldc * cc + gap)
    npdt = c0.A.dtype

    def pack(arrs, stride):
        buf = np.full(stride * batch, np.nan, dtype=npdt)
        for b, a in enumerate(arrs):
            buf[b * stride:b * stride + a.size] = a.reshape(-1)
        return buf
    hA, hB, hC = pack([c.A for c in cases], sA), pack([c.B for c in cases], sB), pack([c.C for c in cases], sC)
    dA, dB, dC = (torch.from_numpy(x).cuda() for x in (hA, hB, hC))
    before = mm.launch_count()
    mm.gemm_strided_batched(dtype, ta, tb, m, n, k, alpha, dA, c0.lda, sA, dB, c0.ldb, sB, beta, dC, c0.ldc, sC,
                            batch, kid)
    launches = mm.launch_count() - before
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    out = dC.cpu().numpy()
    for b, case in enumerate(cases):
        got = out[b * sC:b * sC + case.C.size].reshape(case.C.shape)
        if case.ldc > m:  # padding rows of C keep their bits
            assert np.array_equal(got[:, m:].view(np.uint8), case.C[:, m:].view(np.uint8)), (b, "padding written")
        err = oracle.rel_frobenius(dtype, m, n, np.ascontiguousarray(got), case.ldc, case.reference())
        assert err == err and err <= TOL[dtype], (b, err)
    # the gaps between problems stay untouched (NaN sentinels)
    tail = out.reshape(batch, sC)[:, cases[0].C.size:]
    assert np.isnan(tail.astype(np.float64)).all()
    return launches


@pytest.mark.parametrize("dtype", ["f16", "f32", "f64"])
@pytest.mark.parametrize("ta,tb", MODES)
def test_batched_ragged_one_launch(cuda, mm, oracle, dtype, ta, tb):
    """Ragged shapes x 4 transpose modes x batch 64 through automatic selection: one launch of the
    GEMM kernel (the split-precision fp32 rows add their two split passes)."""
    for (m, n, k, beta) in [(136, 72, 200, 0.5), (257, 130, 65, 0.0)]:
        launches = _batch(cuda, mm, oracle, dtype, ta, tb, m, n, k, 64, 1.0, beta, -1, pad_to=ALIGN[dtype], gap=16)
        assert launches in (1, 3), launches


@pytest.mark.parametrize("dtype,ids", [("f16", [0, 1, 2, 3, 4, 5, 6, 7]), ("f32", [0, 1, 2, 3, 4, 5, 6]), ("f64", [0, 1, 2, 3, 4])])
def test_batched_every_kernel_id(cuda, mm, oracle, dtype, ids):
    for kid in ids:
        launches = _batch(cuda, mm, oracle, dtype, False, True, 200, 136, 96, 5, -1.0, 1.0, kid, pad_to=ALIGN[dtype])
        expect = {("f32", 3): 3, ("f32", 4): 3, ("f32", 5): 3, ("f32", 6): 5}.get((dtype, kid), 1)
        assert launches == expect, (kid, launches)


@pytest.mark.parametrize("dtype", ["f16", "f32", "f64"])
def test_batched_unaligned_strides_fall_back(cuda, mm, oracle, dtype):
    """Leading dimensions and strides TMA cannot take: still correct (fp16 loops over the problems,
    the other dtypes keep one launch through their element-copy paths)."""
    launches = _batch(cuda, mm, oracle, dtype, True, False, 77, 45, 123, 4, 1.0, 0.5, -1, pad_to=None, gap=3)
    assert launches >= 1


def test_batched_64x256cubed_is_faster_than_a_loop(cuda, mm, oracle):
    """64 problems of 256^3 in fp16: one launch whose tile walk covers the batch, against 64 separate calls."""
    torch = cuda
    m = n = k = 256
    batch = 64
    A = torch.randn(batch * m * k, device="cuda").half()
    B = torch.randn(batch * n * k, device="cuda").half()
    C = torch.zeros(batch * m * n, device="cuda").half()

    def batched():
        mm.gemm_strided_batched("f16", False, True, m, n, k, 1.0, A, m, m * k, B, n, n * k, 0.0, C, m, m * n, batch)

    def looped():
        for b in range(batch):
            mm.gemm("f16", False, True, m, n, k, 1.0, A.data_ptr() + 2 * b * m * k, m, B.data_ptr() + 2 * b * n * k, n,
                    0.0, C.data_ptr() + 2 * b * m * n, m)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 10
    t_b, t_l = timed(batched), timed(looped)
    print(f"64 x 256^3 fp16: batched {t_b * 1e3:.1f} us, loop {t_l * 1e3:.1f} us")
    assert t_b * 5 <= t_l, (t_b, t_l)
