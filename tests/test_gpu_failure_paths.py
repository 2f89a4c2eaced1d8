"""Failure paths that can be exercised on a healthy GPU: nothing here faults, traps or hangs the device.

The tcgen05 kernels wait on mbarriers (for a TMA copy, an MMA commit, another warp).  Every such wait is bounded: when
its clock budget runs out the waiting thread raises a host-visible status word, the kernel unwinds and returns, and the
next synchronising call reports B200_ERR_TIMEOUT.  The probe below makes that happen for real with the very same
mbar_wait the kernels use -- one warp, no tensor memory, no copy in flight, a barrier nobody completes -- after the
budget has been shortened to a millisecond, and then checks that the context is still healthy.
"""
import time

import numpy as np
import pytest

from conftest import assert_close
from oracle import pt_matrix

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_the_context_stays_usable(oracle):
    from callaghandev.ml_b200 import GEMM_TF32_TCGEN05, B200Error, CudaB200AccelerationManager, _lib

    m = CudaB200AccelerationManager(0, GEMM_TF32_TCGEN05)
    if not m.has_tcgen05():
        m.Dispose()
        pytest.skip("device is not compute capability 10.x")
    a, b = pt_matrix(256, 256, 1), pt_matrix(256, 256, 2)
    want = oracle.MatrixMultiply(a, b)
    assert_close(want, m.MatrixMultiply(a, b), 2e-3, "GEMM before the probe")
    m.set_wait_budget_us(1000)
    try:
        t0 = time.perf_counter()
        rc = m.lib.b200_probe_wait_timeout(m.ctx)
        dt = time.perf_counter() - t0
        assert rc == _lib.ERR_TIMEOUT, f"expected the timeout status, got {rc}"
        assert b"wait" in m.lib.b200_last_error(m.ctx)
        assert dt < 1.0, f"the wait must give up after about a millisecond, took {dt:.3f} s"
        with pytest.raises(B200Error):  # the same through the exception mapping of the host mirror
            m.probe_wait_timeout()
        # the status was delivered once; the context and the tensor-core kernels work as before
        m.synchronize()
        assert_close(want, m.MatrixMultiply(a, b), 2e-3, "GEMM after the probe")
    finally:
        m.set_wait_budget_us(2_000_000)
    assert_close(want, m.MatrixMultiply(a, b), 2e-3, "GEMM with the default budget restored")
    with pytest.raises(IndexError):
        m.set_wait_budget_us(0)
    m.Dispose()
