"""Pins the oracle's sig_coef: each coefficient equals the matching entry of the oracle's full
signature (itself pinned by the reference's golden vectors), with and without the path
transforms and prefixes; the backward pass agrees with central finite differences."""
import numpy as np
import pytest

from oracle import oracle

WORDS = [(0,), (1, 0), (2, 2, 1), (0, 1, 2, 0), (), (1, 1)]


def _idx(word, dim):
    i = 0
    for letter in word:
        i = i * dim + letter + 1
    return i


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("flags", [(False, False), (True, False), (False, True), (True, True)])
def test_coefficients_are_entries_of_the_signature(dtype, flags):
    ta, ll = flags
    rng = np.random.default_rng(0)
    path = (rng.standard_normal((3, 7, 3)).cumsum(1) * 0.4).astype(dtype)
    dim = (6 if ll else 3) + (1 if ta else 0)
    full = oracle.sig(path, 4, time_aug=ta, lead_lag=ll, end_time=1.5, scalar_term=True)
    got = oracle.sig_coef(path, WORDS, time_aug=ta, lead_lag=ll, end_time=1.5)
    want = full[:, [_idx(w, dim) for w in WORDS]]
    tol = dict(rtol=1e-11, atol=1e-13) if dtype == np.float64 else dict(rtol=2e-4, atol=1e-5)
    np.testing.assert_allclose(got, want, **tol)
    pre = oracle.sig_coef(path, WORDS, time_aug=ta, lead_lag=ll, end_time=1.5, prefixes=True)
    expect = [w[:k] for w in WORDS for k in (range(1, len(w) + 1) if w else [0])]
    np.testing.assert_allclose(pre, full[:, [_idx(w, dim) for w in expect]], **tol)


def test_short_paths():
    np.testing.assert_array_equal(oracle.sig_coef(np.zeros((1, 2)), [(0,), (), (1, 0)], prefixes=True), [0, 1, 0, 0])


@pytest.mark.parametrize("flags", [(False, False), (True, False), (False, True), (True, True)])
def test_backprop_matches_finite_differences(flags):
    ta, ll = flags
    rng = np.random.default_rng(1)
    path = rng.standard_normal((2, 5, 2)).cumsum(1) * 0.5
    dim = (4 if ll else 2) + (1 if ta else 0)
    words = [(0,), (1, 0), (dim - 1, 0, 1), (), (1, 1, dim - 1, 0)]
    kw = dict(time_aug=ta, lead_lag=ll, end_time=0.8)
    coefs = oracle.sig_coef(path, words, prefixes=True, **kw)
    w = rng.standard_normal(coefs.shape)
    got = oracle.sig_coef_backprop(path, words, coefs, w, **kw)
    want = np.zeros_like(path)
    eps = 1e-6
    for i in range(path.size):
        hi, lo = path.copy().reshape(-1), path.copy().reshape(-1)
        hi[i] += eps
        lo[i] -= eps
        f = lambda x: float((w * oracle.sig_coef(x.reshape(path.shape), words, prefixes=True, **kw)).sum())
        want.reshape(-1)[i] = (f(hi) - f(lo)) / (2 * eps)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-8)
