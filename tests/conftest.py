import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def assert_close(expected, actual, tol, label=""):
    """The reference's own parity metric: |exp-act| <= tol*max(1,|exp|), NaN==NaN, inf must match exactly
    (CallaghanDev.ML.TestConsoleApp/Tests/AccelerationManagerParityTests.cs:1923-1936)."""
    e = np.asarray(expected, dtype=np.float64)
    a = np.asarray(actual, dtype=np.float64)
    assert e.shape == a.shape, f"{label}: shape {e.shape} vs {a.shape}"
    both_nan = np.isnan(e) & np.isnan(a)
    inf = np.isinf(e) | np.isinf(a)
    ok_inf = ~inf | (e == a)
    with np.errstate(invalid="ignore"):
        diff = np.abs(e - a)
        bound = tol * np.maximum(1.0, np.abs(e))
        ok = both_nan | (inf & ok_inf) | (~inf & (diff <= bound))
    if not ok.all():
        idx = np.unravel_index(np.argmax(np.where(ok, 0, np.nan_to_num(diff, nan=np.inf, posinf=np.inf))), e.shape) if e.shape else ()
        raise AssertionError(f"{label}: {int((~ok).sum())}/{e.size} outside tol {tol}; worst at {idx}: expected {e[idx]}, got {a[idx]}")


def assert_tensor_close(expected, actual, tol, label="", quantum=None, ref_max=None, ref_l2=None):
    """Per-tensor normalised bound for whole-network quantities (gradients, weight updates), whose elements are far
    below 1 so that the operator metric above would be an absolute bound:
        max|exp-act| <= tol*max|exp|   and   ||exp-act||_2 <= tol*||exp||_2.
    `quantum` (same shape, or a scalar) is an additive per-element allowance for a quantity that both sides round
    to a grid before it can be observed: a weight update is only visible as w_after - w_before, and w_after is
    rounded to FP32, so two correct implementations may differ by one unit in the last place of the weight.
    ref_max / ref_l2 replace the tensor's own magnitude as the yardstick (for a tensor that is the small remainder of
    cancelling contributions, whose error is set by the size of what cancels)."""
    e = np.asarray(expected, dtype=np.float64).reshape(-1)
    a = np.asarray(actual, dtype=np.float64).reshape(-1)
    assert e.shape == a.shape, f"{label}: shape {e.shape} vs {a.shape}"
    assert np.isfinite(a).all(), f"{label}: non-finite values"
    q = np.zeros_like(e) if quantum is None else np.broadcast_to(np.asarray(quantum, np.float64).reshape(-1), e.shape)
    diff = np.abs(e - a)
    ref_max = (float(np.max(np.abs(e))) if e.size else 0.0) if ref_max is None else float(ref_max)
    ref_l2 = float(np.sqrt((e * e).sum())) if ref_l2 is None else float(ref_l2)
    excess = diff - q
    worst = int(np.argmax(excess)) if e.size else 0
    if e.size and excess[worst] > tol * ref_max:
        raise AssertionError(f"{label}: max|diff| {diff[worst]:.3e} at {worst} (expected {e[worst]:.6e}, got {a[worst]:.6e}) "
                             f"> {tol:g} x max|ref| {ref_max:.3e} = {diff[worst] / max(ref_max, 1e-300):.2e} relative")
    l2 = float(np.sqrt((np.maximum(excess, 0.0) ** 2).sum()))
    if l2 > tol * ref_l2:
        raise AssertionError(f"{label}: ||diff||_2 {l2:.3e} > {tol:g} x ||ref||_2 {ref_l2:.3e} = {l2 / max(ref_l2, 1e-300):.2e} relative")
    return (float(diff.max()) / ref_max if ref_max else 0.0)


def ulp32(x):
    """Spacing of FP32 at |x| (what one rounding of a stored weight can move it by)."""
    return np.spacing(np.abs(np.asarray(x, np.float32))).astype(np.float64)


@pytest.fixture(scope="session")
def oracle():
    from oracle import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def oracle64():
    from oracle import Oracle

    return Oracle(f64=True)
