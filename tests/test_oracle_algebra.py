"""Pins the oracle's tensor exponential, correction variants, linear signature and sig_join.

Known answers are the ones written out in the reference's own tests
(tests/test_signature.py:126-188); the identities are the ones its tests check
(tests/test_linear_and_branched_join.py:86-112, tests/test_signature.py:113-123,151-177);
backward passes are checked against central finite differences in float64.
"""
import numpy as np
import pytest

from oracle import oracle


def _fd_grad(f, x, eps=1e-6):
    g = np.zeros_like(x)
    flat, gf = x.reshape(-1), g.reshape(-1)
    for i in range(flat.size):
        old = flat[i]
        flat[i] = old + eps
        hi = f(x)
        flat[i] = old - eps
        lo = f(x)
        flat[i] = old
        gf[i] = (hi - lo) / (2 * eps)
    return g


def test_correction_single_segment_known_answer():
    # exp(3 e1 + 2 e11), truncated at level 4 (reference tests/test_signature.py:126-136)
    path = np.array([[0.0], [3.0]])
    out = oracle.sig(path, 4, scalar_term=True, correction=np.array([2.0]))
    np.testing.assert_allclose(out, [1.0, 3.0, 6.5, 10.5, 14.375], rtol=1e-14)


def test_correction_propagates_across_segments_known_answer():
    # two zero increments, each with level-2 correction 2 (reference tests/test_signature.py:138-148)
    out = oracle.sig(np.zeros((3, 1)), 3, scalar_term=True, correction=np.array([2.0]))
    np.testing.assert_allclose(out, [1.0, 0.0, 4.0, 0.0], atol=1e-15)


def test_correction_time_aug_known_answer():
    # correction lives on the data channel; the time channel gets none (reference tests/test_signature.py:179-188)
    out = oracle.sig(np.zeros((2, 1)), 2, time_aug=True, scalar_term=True, correction=np.array([[2.0]]))
    np.testing.assert_allclose(out, [1.0, 0.0, 1.0, 2.0, 0.0, 0.0, 0.5], atol=1e-15)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_zero_correction_is_plain_signature(dtype):
    rng = np.random.default_rng(0)
    path = rng.standard_normal((3, 9, 3)).astype(dtype).cumsum(1) * 0.3
    plain = oracle.sig(path, 4)
    corrected = oracle.sig(path, 4, correction=np.zeros(9, dtype=dtype))
    tol = 1e-5 if dtype == np.float32 else 1e-12
    np.testing.assert_allclose(corrected, plain, rtol=tol, atol=tol)


def test_correction_layouts_agree():
    rng = np.random.default_rng(1)
    path = rng.standard_normal((2, 4, 2)).cumsum(1)
    const = rng.standard_normal(4 + 8) * 0.2
    shared = rng.standard_normal((3, 4)) * 0.2
    a = oracle.sig(path, 3, scalar_term=True, correction=const)
    b = oracle.sig(path, 3, scalar_term=True, correction=np.broadcast_to(const, (2, 3, 12)).copy())
    np.testing.assert_allclose(a, b, rtol=1e-14)
    a = oracle.sig(path, 3, correction=shared)
    b = oracle.sig(path, 3, correction=np.broadcast_to(shared, (2, 3, 4)).copy())
    np.testing.assert_allclose(a, b, rtol=1e-14)


def test_tensor_exp_of_level_one_element_is_linear_signature():
    rng = np.random.default_rng(2)
    v = rng.standard_normal(3)
    n = oracle.sig_length(3, 5, True)
    x = np.zeros(n)
    x[1:4] = v
    np.testing.assert_allclose(oracle.tensor_exp(x, 3, 5), oracle.linear_sig(v, 5, scalar_term=True), rtol=1e-13)


def test_tensor_exp_backprop_matches_finite_differences():
    rng = np.random.default_rng(3)
    dim, degree = 2, 4
    n = oracle.sig_length(dim, degree, True)
    x = rng.standard_normal(n) * 0.4
    x[0] = 0.0
    w = rng.standard_normal(n)
    w[0] = 0.0
    got = oracle.tensor_exp_backprop(w, x, dim, degree)
    want = _fd_grad(lambda y: float(np.dot(w, oracle.tensor_exp(y, dim, degree))), x.copy())
    np.testing.assert_allclose(got[1:], want[1:], rtol=1e-6, atol=1e-8)


@pytest.mark.parametrize("time_aug", [False, True])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_correction_backprop_matches_finite_differences(time_aug, scalar_term):
    rng = np.random.default_rng(4)
    path = rng.standard_normal((2, 5, 2)).cumsum(1) * 0.5
    corr = rng.standard_normal((2, 4, 4)) * 0.3
    kw = dict(time_aug=time_aug, correction=corr)
    s = oracle.sig(path, 3, scalar_term=scalar_term, **kw)
    w = rng.standard_normal(s.shape)
    got = oracle.sig_backprop(path, s, w, 3, **kw)
    want = _fd_grad(lambda p: float((w * oracle.sig(p, 3, scalar_term=scalar_term, **kw)).sum()), path.copy())
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("prepend", [False, True])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_sig_join_is_signature_of_extended_path(prepend, scalar_term):
    rng = np.random.default_rng(5)
    path = rng.standard_normal((3, 6, 3)).cumsum(1) * 0.4
    v = rng.standard_normal((3, 3)) * 0.5
    s = oracle.sig(path, 4, scalar_term=scalar_term)
    joined = oracle.sig_join(s, v, 3, 4, prepend=prepend)
    if prepend:
        ext = np.concatenate([path[:, :1] - v[:, None], path], axis=1)
    else:
        ext = np.concatenate([path, path[:, -1:] + v[:, None]], axis=1)
    np.testing.assert_allclose(joined, oracle.sig(ext, 4, scalar_term=scalar_term), rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("prepend", [False, True])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_sig_join_backprop_matches_finite_differences(prepend, scalar_term):
    rng = np.random.default_rng(6)
    dim, degree = 2, 3
    s = oracle.sig(rng.standard_normal((2, 5, dim)).cumsum(1) * 0.5, degree, scalar_term=scalar_term)
    v = rng.standard_normal((2, dim)) * 0.6
    w = rng.standard_normal(s.shape)
    d_sig, d_disp = oracle.sig_join_backprop(w, s, v, dim, degree, prepend=prepend)
    loss_s = lambda x: float((w * oracle.sig_join(x, v, dim, degree, prepend=prepend)).sum())
    loss_v = lambda x: float((w * oracle.sig_join(s, x, dim, degree, prepend=prepend)).sum())
    want_sig = _fd_grad(loss_s, s.copy())
    if scalar_term:
        want_sig[:, 0] = 0.0  # the scalar slot carries no gradient (cp_sig_join.h:213)
    np.testing.assert_allclose(d_sig, want_sig, rtol=1e-6, atol=1e-8)
    np.testing.assert_allclose(d_disp, _fd_grad(loss_v, v.copy()), rtol=1e-6, atol=1e-8)


def test_linear_sig_levels():
    v = np.array([2.0, -1.0])
    out = oracle.linear_sig(v, 3)
    np.testing.assert_allclose(out[:2], v)
    np.testing.assert_allclose(out[2:6], np.outer(v, v).reshape(-1) / 2)
    np.testing.assert_allclose(out[6:], np.einsum("i,j,k->ijk", v, v, v).reshape(-1) / 6)
