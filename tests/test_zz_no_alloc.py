"""The SGEMM entry point that allocates nothing (mmbo_gemm_f32_noalloc).

It exists for callers that cannot call cudaMalloc when they need a GEMM: latency-critical
loops where an allocation may stall the whole device, plugins inside a host application
that owns all device memory, processes whose pool is already full.  Its scratch is a
fixed 32 MiB array inside the library's device image instead of heap memory.

The test calls it through the C ABI twice in a row, with different operands, and
compares each result with what the existing entry point (mmbo_gemm_f32, the same
split-precision kernel with library-managed scratch) returns for the same inputs --
relative Frobenius error within the fp32 tolerance of the other tests (1e-5) -- and
with the CPU oracle.  The second call also proves that the scratch contents left behind
by the first call do no harm.  Problems beyond the built-in scratch are refused.

This file sorts last so that a run stopping at the first failure has already run
every other test; it passes on its own in a fresh process as well.
"""
import ctypes

import numpy as np
import pytest

from helpers import Case, to_device

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _noalloc(lib, case, dA, dB, dC):
    a, b = ctypes.c_float(case.alpha), ctypes.c_float(case.beta)
    return lib.mmbo_gemm_f32_noalloc(int(case.ta), int(case.tb), case.m, case.n, case.k, ctypes.byref(a),
                                     dA.data_ptr(), case.lda, dB.data_ptr(), case.ldb, ctypes.byref(b),
                                     dC.data_ptr(), case.ldc, None)


def test_noalloc_matches_existing_entry_point_twice_in_a_row(cuda, mm, oracle):
    torch = cuda
    from gemm_mmbo_b200._lib import LIB
    calls = [Case(oracle, "f32", False, True, 520, 392, 328, 1.5, -0.25, pad=(3, 3, 3), seed=11),
             Case(oracle, "f32", True, False, 300, 777, 1000, 1.0, 0.0, pad=(0, 4, 1), seed=12, c_poison=True)]
    free_after = []
    for case in calls:
        _, dA = to_device(torch, case.A)
        _, dB = to_device(torch, case.B)
        _, dC_new = to_device(torch, case.C)
        _, dC_old = to_device(torch, case.C)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _noalloc(LIB, case, dA, dB, dC_new)
        assert rc == 0, mm.status_string(rc)
        torch.cuda.synchronize()
        free_after.append((free_before, torch.cuda.mem_get_info()[0]))
        mm.gemm("f32", case.ta, case.tb, case.m, case.n, case.k, case.alpha, dA, case.lda, dB, case.ldb, case.beta,
                dC_old, case.ldc, 4)
        torch.cuda.synchronize()
        assert mm.device_status() == 0
        new = dC_new.cpu().numpy().reshape(case.C.shape)
        old = dC_old.cpu().numpy().reshape(case.C.shape)
        win_new = new[:, :case.m].astype(np.float64)
        win_old = old[:, :case.m].astype(np.float64)
        rel = np.linalg.norm(win_new - win_old) / np.linalg.norm(win_old)
        assert rel <= TOL, rel
        # padding rows of C untouched, and the oracle agrees as well
        if case.ldc > case.m:
            assert np.array_equal(new[:, case.m:].view(np.uint32), case.C[:, case.m:].view(np.uint32))
        err = oracle.rel_frobenius("f32", case.m, case.n, np.ascontiguousarray(new), case.ldc, case.reference())
        assert err <= TOL, err
    # The property in the name: free device memory is the same before and after a call.  The very
    # first call of a process may make the driver load the kernels' code, so it is the second
    # (warm) call that is held to it.
    before, after = free_after[1]
    assert after == before, f"device memory changed across a warm call: {before} -> {after}"


def test_noalloc_refuses_problems_beyond_its_scratch(cuda, mm):
    from gemm_mmbo_b200._lib import LIB
    one = ctypes.c_float(1.0)
    big = 4096  # 8 * (m + n) * k = 256 MiB > 32 MiB
    buf = cuda.empty(16, dtype=cuda.float32, device="cuda")  # never dereferenced: refused before any launch
    rc = LIB.mmbo_gemm_f32_noalloc(0, 0, big, big, big, ctypes.byref(one), buf.data_ptr(), big, buf.data_ptr(), big,
                                   ctypes.byref(one), buf.data_ptr(), big, None)
    assert rc == -16
    assert "scratch" in mm.status_string(rc)
