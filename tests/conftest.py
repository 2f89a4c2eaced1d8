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


@pytest.fixture(scope="session")
def oracle():
    from oracle import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def oracle64():
    from oracle import Oracle

    return Oracle(f64=True)
