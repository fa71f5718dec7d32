import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden", "reference_sig_vectors.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN)


def brownian_paths(seed, batch, length, dim, dtype=np.float64):
    """Cumulative sums of N(0, 1/L) increments starting at 0 (the benchmark's input law)."""
    rng = np.random.default_rng(seed)
    inc = rng.normal(0.0, np.sqrt(1.0 / length), (batch, length - 1, dim))
    path = np.concatenate([np.zeros((batch, 1, dim)), np.cumsum(inc, axis=1)], axis=1)
    return np.ascontiguousarray(path.astype(dtype))


def level_slices(dim, degree, scalar_term=False):
    """[(level, slice)] of a flat signature."""
    out, start = [], 1 if scalar_term else 0
    for k in range(1, degree + 1):
        out.append((k, slice(start, start + dim ** k)))
        start += dim ** k
    return out


def assert_sig_close(actual, expected, dim, degree, rtol, scalar_term=False, what="sig"):
    """Per-coefficient relative check with a per-level floor.

    |a - b| <= rtol * max(|b|, floor_k) where floor_k is the largest magnitude of
    level k in that path: coefficients that are small only through cancellation
    are compared on the scale of their level.
    """
    actual = np.asarray(actual, dtype=np.float64).reshape(-1, actual.shape[-1])
    expected = np.asarray(expected, dtype=np.float64).reshape(-1, expected.shape[-1])
    assert actual.shape == expected.shape, (actual.shape, expected.shape)
    if scalar_term:
        np.testing.assert_allclose(actual[:, 0], expected[:, 0], rtol=rtol)
    for k, sl in level_slices(dim, degree, scalar_term):
        a, b = actual[:, sl], expected[:, sl]
        floor = np.abs(b).max(axis=1, keepdims=True)
        err = np.abs(a - b) / np.maximum(np.maximum(np.abs(b), floor), 1e-300)
        worst = err.max() if err.size else 0.0
        assert worst <= rtol, "%s level %d: max scaled rel err %.3e > %.1e" % (what, k, worst, rtol)


def assert_grad_close(actual, expected, rtol, what="grad"):
    """|a - b| <= rtol * max(|b|, largest |b| of that path)."""
    a = np.asarray(actual, dtype=np.float64)
    b = np.asarray(expected, dtype=np.float64)
    assert a.shape == b.shape
    a = a.reshape(-1, a.shape[-2] * a.shape[-1]) if a.ndim >= 2 else a[None]
    b = b.reshape(a.shape)
    floor = np.abs(b).max(axis=1, keepdims=True)
    err = np.abs(a - b) / np.maximum(np.maximum(np.abs(b), floor), 1e-300)
    worst = err.max() if err.size else 0.0
    assert worst <= rtol, "%s: max scaled rel err %.3e > %.1e" % (what, worst, rtol)


def assert_grad_parity(actual, oracle_same_dtype, oracle_f64, rtol, what="grad"):
    """Gradient parity.  float64: per-coefficient relative check against the oracle.
    float32: the reverse sweep subtracts increment gradients that can be orders of
    magnitude larger than the result, so two correct float32 implementations differ by
    rounding noise on the scale of those intermediates.  The check is then twofold: close
    to the float32 oracle up to that noise, and no less accurate than it when both are
    measured against the float64 oracle (error <= 3x the oracle's own float32 error + rtol)."""
    a = np.asarray(actual, dtype=np.float64)
    if np.asarray(actual).dtype == np.float64:
        assert_grad_close(a, oracle_same_dtype, rtol, what)
        return
    truth = np.asarray(oracle_f64, dtype=np.float64).reshape(a.shape[0], -1)
    ref32 = np.asarray(oracle_same_dtype, dtype=np.float64).reshape(a.shape[0], -1)
    a = a.reshape(a.shape[0], -1)
    floor = np.maximum(np.abs(truth).max(axis=1, keepdims=True), 1e-300)
    err_ours = (np.abs(a - truth) / floor).max()
    err_ref = (np.abs(ref32 - truth) / floor).max()
    assert err_ours <= 3 * err_ref + rtol, "%s: float32 error %.3e vs reference-order float32 error %.3e" % (
        what, err_ours, err_ref)
