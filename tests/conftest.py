import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


# Parity tolerances: 1e-12 relative for f64 and 1e-5 for f32. Outputs are signed sums of
# up to thousands of terms and some land near zero, so "relative" is taken against the
# largest magnitude of the tensor (norm-wise), plus an element-wise allclose whose
# absolute floor is that same quantity.
TOL = {np.dtype("float64"): 1e-12, np.dtype("float32"): 1e-5}


def assert_parity(actual, expected, what="", tol=None):
    actual = np.asarray(actual)
    expected = np.asarray(expected)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} != {expected.shape}"
    assert actual.dtype == expected.dtype, f"{what}: dtype {actual.dtype} != {expected.dtype}"
    if expected.size == 0:
        return
    tol = TOL[expected.dtype] if tol is None else tol
    scale = float(np.max(np.abs(expected)))
    err = float(np.max(np.abs(actual.astype(np.float64) - expected.astype(np.float64))))
    assert np.isfinite(actual).all(), f"{what}: non-finite values"
    assert err <= tol * max(scale, 1e-300), f"{what}: max|diff|={err:.3e} > {tol:g}*{scale:.3e}"
    assert np.allclose(actual, expected, rtol=tol * 1e3, atol=tol * scale), what


@pytest.fixture(scope="session")
def oracle():
    from oracle.mops_oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle.mops_oracle import Reference, have_reference
    if not have_reference():
        pytest.skip("oracle/_ref/libmops_ref.so not built (reference tree not mounted)")
    return Reference()
