"""Shared machinery of the GPU parity tests: build seeded operands with the oracle's
generator, run the library through its C ABI on device copies surrounded by guard
bands, and compare with the oracle."""
from __future__ import annotations

import numpy as np

GUARD = 256  # elements of sentinel before and after every device buffer

TOL = {"f32": 1e-5, "f16": 2e-3, "f64": 1e-13}  # relative Frobenius error (fp32/fp16: BASELINE north_star)


def lead_dims(ta, tb, m, n, k):
    """Leading extents (rows of the stored arrays) of A, B, C."""
    return (k if ta else m), (n if tb else k), m


def stored_cols(ta, tb, m, n, k):
    return (m if ta else k), (k if tb else n), n


class Case:
    def __init__(self, O, dtype, ta, tb, m, n, k, alpha, beta, pad=(0, 0, 0), seed=1234,
                 dist=None, scale=1.0, c_poison=False):
        self.O, self.dtype, self.ta, self.tb = O, dtype, ta, tb
        self.m, self.n, self.k, self.alpha, self.beta = m, n, k, alpha, beta
        ra, rb, rc = lead_dims(ta, tb, m, n, k)
        ca, cb, cc = stored_cols(ta, tb, m, n, k)
        self.lda, self.ldb, self.ldc = max(ra + pad[0], 1), max(rb + pad[1], 1), max(rc + pad[2], 1)
        dist = O.DIST_UNIFORM if dist is None else dist
        self.A = O.fill(dtype, ra, ca, self.lda, seed=seed, mat=O.MAT_A, dist=dist, scale=scale)
        self.B = O.fill(dtype, rb, cb, self.ldb, seed=seed, mat=O.MAT_B, dist=dist, scale=scale)
        self.C = O.fill(dtype, rc, cc, self.ldc, seed=seed, mat=O.MAT_C, dist=dist, scale=scale)
        if c_poison:  # beta == 0 must not read C: poison the whole window
            self.C[:, :] = np.nan

    def reference(self):
        return self.O.gemm(self.dtype, self.ta, self.tb, self.m, self.n, self.k, self.alpha, self.A,
                           self.lda, self.B, self.ldb, self.beta, self.C, self.ldc)


def to_device(torch, host: np.ndarray):
    """Device copy of a host array inside a larger buffer with sentinel guard bands.
    Returns (whole buffer, view of the payload)."""
    flat = torch.from_numpy(host.reshape(-1))
    buf = torch.empty(flat.numel() + 2 * GUARD, dtype=flat.dtype, device="cuda")
    buf.fill_(float("nan"))
    buf[GUARD:GUARD + flat.numel()].copy_(flat)
    return buf, buf[GUARD:GUARD + flat.numel()]


def bits(a: np.ndarray) -> np.ndarray:
    return a.view({2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


def run_and_check(torch, mm, case: Case, kernel_id=-1, tol=None, ref=None):
    """Runs the library on `case`; asserts guard bands and padding rows are untouched and
    the result is within tolerance of the oracle.  Returns the relative Frobenius error."""
    O = case.O
    bufA, dA = to_device(torch, case.A)
    bufB, dB = to_device(torch, case.B)
    bufC, dC = to_device(torch, case.C)
    mm.gemm(case.dtype, case.ta, case.tb, case.m, case.n, case.k, case.alpha, dA, case.lda, dB, case.ldb,
            case.beta, dC, case.ldc, kernel_id)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    outC = bufC.cpu().numpy()
    got = outC[GUARD:GUARD + case.C.size].reshape(case.C.shape)
    # guard bands (NaN sentinels have one bit pattern) and inputs untouched
    sent = bits(np.full(1, np.nan, dtype=case.C.dtype))[0]
    assert (bits(outC[:GUARD]) == sent).all() and (bits(outC[-GUARD:]) == sent).all(), "C guard band written"
    assert np.array_equal(bits(bufA.cpu().numpy()[GUARD:GUARD + case.A.size]), bits(case.A.reshape(-1)))
    assert np.array_equal(bits(bufB.cpu().numpy()[GUARD:GUARD + case.B.size]), bits(case.B.reshape(-1)))
    # padding rows of C (row >= m) keep their bits
    if case.ldc > case.m and case.n > 0:
        assert np.array_equal(bits(got[:, case.m:]), bits(case.C[:, case.m:])), "C padding rows written"
    if case.m == 0 or case.n == 0:
        return 0.0
    ref = case.reference() if ref is None else ref
    err = O.rel_frobenius(case.dtype, case.m, case.n, np.ascontiguousarray(got), case.ldc, ref)
    tol = TOL[case.dtype] if tol is None else tol
    assert err == err and err <= tol, f"rel Frobenius {err:.3e} > {tol:.1e}"
    return err
