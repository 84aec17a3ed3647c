"""Failure detection without faulting the GPU: a kernel whose barrier wait can never
complete must give up after its limit, record a fault code the host can read, and leave
the context usable for the next launch."""
import ctypes
import time

import pytest

from helpers import Case, run_and_check

pytestmark = pytest.mark.gpu


def test_bounded_wait_times_out_and_reports(cuda, mm, oracle):
    from gemm_mmbo_b200._lib import LIB
    assert mm.device_status() == 0
    t0 = time.perf_counter()
    assert LIB.mmbo_selftest_bounded_wait(5_000_000, None) == 0  # 5 ms limit
    status = ctypes.c_uint32()
    rc = LIB.mmbo_device_status(ctypes.byref(status))
    elapsed = time.perf_counter() - t0
    assert rc == -13                      # MMBO_ERR_DEVICE_FAULT
    assert status.value >> 24 == 7        # kFaultWaitPeer
    assert status.value & 0xffffff == 0x5e1f
    assert elapsed < 2.0                  # the wait ran out on its own
    assert "time-out" in mm.status_string(rc)
    # the word is cleared by the read and the context still works
    assert mm.device_status() == 0
    run_and_check(cuda, mm, Case(oracle, "f16", False, True, 264, 136, 72, 1.0, 0.5), -1)


def test_selftest_rejects_long_limits(cuda, mm):
    from gemm_mmbo_b200._lib import LIB
    assert LIB.mmbo_selftest_bounded_wait(0, None) == -2
    assert LIB.mmbo_selftest_bounded_wait(5_000_000_000, None) == -2
