"""Pins the oracle's signature -> log-signature map (expanded and Lyndon-word coordinates).

Closed forms and identities (the reference's golden vectors are checked in
test_oracle_log_golden.py): the logarithm of a straight segment's signature is the segment,
level 2 is S_2 - S_1 (x) S_1 / 2, exp(log S) = S through the oracle's tensor exponential, the
number of Lyndon coordinates is Witt's necklace count (pysiglib/sig_length.py:97-163), and the
backward pass agrees with central finite differences."""
import numpy as np
import pytest

from oracle import oracle


def _witt(d, n):
    def mobius(k):
        res, p = 1, 2
        while p * p <= k:
            if k % p == 0:
                k //= p
                if k % p == 0:
                    return 0
                res = -res
            p += 1
        return -res if k > 1 else res
    return sum(sum(mobius(i // x) * d ** x for x in range(1, i + 1) if i % x == 0) // i for i in range(1, n + 1))


@pytest.mark.parametrize("d,n", [(1, 4), (2, 3), (2, 6), (3, 4), (5, 3)])
def test_lyndon_count_and_order(d, n):
    idx = oracle.lyndon_indices(d, n)
    assert len(idx) == _witt(d, n) == oracle.log_sig_length(d, n)
    if (d, n) == (2, 3):
        # words 0, 1, 01, 001, 011 at positions 1, 2, 4, 8, 10 of the signature with its scalar slot
        assert idx.tolist() == [1, 2, 4, 8, 10]


def test_log_of_a_straight_segment_is_the_segment():
    v = np.array([0.3, -1.2, 0.7])
    s = oracle.linear_sig(v, 5, scalar_term=True)
    log = oracle.sig_to_log_sig(s, 3, 5, method=0)
    np.testing.assert_allclose(log[1:4], v, rtol=1e-15)
    np.testing.assert_allclose(log[4:], 0, atol=1e-15)
    assert log[0] == 0
    np.testing.assert_allclose(oracle.sig_to_log_sig(s, 3, 5, method=1)[:3], v, rtol=1e-15)


@pytest.mark.parametrize("scalar_term", [False, True])
def test_level_two_closed_form_and_exp_round_trip(scalar_term):
    rng = np.random.default_rng(0)
    path = rng.standard_normal((3, 8, 3)).cumsum(1) * 0.4
    s = oracle.sig(path, 4, scalar_term=scalar_term)
    log = oracle.sig_to_log_sig(s, 3, 4, method=0)
    assert log.shape == s.shape
    off = 1 if scalar_term else 0
    s1, s2 = s[:, off:off + 3], s[:, off + 3:off + 12]
    np.testing.assert_allclose(log[:, off:off + 3], s1, rtol=1e-15)
    np.testing.assert_allclose(log[:, off + 3:off + 12], s2 - np.einsum("bi,bj->bij", s1, s1).reshape(3, 9) / 2,
                               rtol=1e-12, atol=1e-14)
    full_log = log if scalar_term else np.concatenate([np.zeros((3, 1)), log], axis=1)
    for b in range(3):
        back = oracle.tensor_exp(full_log[b], 3, 4)
        np.testing.assert_allclose(back[1:], s[b, off:], rtol=1e-11, atol=1e-13)
    lyndon = oracle.sig_to_log_sig(s, 3, 4, method=1)
    idx = oracle.lyndon_indices(3, 4).astype(np.int64)
    np.testing.assert_array_equal(lyndon, full_log[:, idx])


@pytest.mark.parametrize("method", [0, 1])
@pytest.mark.parametrize("scalar_term", [False, True])
@pytest.mark.parametrize("d,n", [(2, 2), (2, 4), (3, 3), (2, 5)])
def test_backprop_matches_finite_differences(method, scalar_term, d, n):
    rng = np.random.default_rng(d * 10 + n)
    s = oracle.sig(rng.standard_normal((2, 6, d)).cumsum(1) * 0.5, n, scalar_term=scalar_term)
    out = oracle.sig_to_log_sig(s, d, n, method=method)
    w = rng.standard_normal(out.shape)
    got = oracle.sig_to_log_sig_backprop(s, w, d, n, method=method)
    want = np.zeros_like(s)
    eps = 1e-6
    for i in range(s.size):
        hi, lo = s.copy().reshape(-1), s.copy().reshape(-1)
        hi[i] += eps
        lo[i] -= eps
        f = lambda x: float((w * oracle.sig_to_log_sig(x.reshape(s.shape), d, n, method=method)).sum())
        want.reshape(-1)[i] = (f(hi) - f(lo)) / (2 * eps)
    if scalar_term:
        want[:, 0] = 0  # the scalar slot is a constant of the map (cp_tensor_log.h:190-191)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-8)


def _word_index(word, dim):
    i = 0
    for letter in word:
        i = i * dim + letter + 1
    return i


@pytest.mark.parametrize("d,n", [(2, 3), (2, 6), (3, 4), (4, 3)])
def test_lyndon_basis_coordinates_rebuild_the_expanded_logarithm(d, n):
    # method 2 pins itself: sum_j b_j [w_j], expanded word by word, must be the whole tensor logarithm
    rng = np.random.default_rng(d + n)
    s = oracle.sig(rng.standard_normal((2, 7, d)).cumsum(1) * 0.5, n, scalar_term=True)
    full = oracle.sig_to_log_sig(s, d, n, method=0)
    basis = oracle.sig_to_log_sig(s, d, n, method=2)
    words, exps = oracle.lyndon_bracket_expansions(d, n)
    assert basis.shape == (2, len(words))
    rebuilt = np.zeros_like(full)
    for j, e in enumerate(exps):
        for w, c in e.items():
            rebuilt[:, _word_index(w, d)] += c * basis[:, j]
    np.testing.assert_allclose(rebuilt, full, rtol=1e-9, atol=1e-12)
    P = oracle.lyndon_projection(d, n)
    assert np.allclose(np.diag(P), 1) and np.allclose(np.triu(P, 1), 0)
    if (d, n) == (2, 3):
        np.testing.assert_array_equal(P, np.eye(5))  # brackets 0, 1, [0,1], [0,[0,1]], [[0,1],1]


@pytest.mark.parametrize("d,n", [(2, 5), (3, 4)])
def test_lyndon_basis_backprop_matches_finite_differences(d, n):
    rng = np.random.default_rng(d * 7 + n)
    s = oracle.sig(rng.standard_normal((1, 6, d)).cumsum(1) * 0.5, n)
    out = oracle.sig_to_log_sig(s, d, n, method=2)
    w = rng.standard_normal(out.shape)
    got = oracle.sig_to_log_sig_backprop(s, w, d, n, method=2)
    want = np.zeros_like(s)
    eps = 1e-6
    for i in range(s.size):
        hi, lo = s.copy().reshape(-1), s.copy().reshape(-1)
        hi[i] += eps
        lo[i] -= eps
        f = lambda x: float((w * oracle.sig_to_log_sig(x.reshape(s.shape), d, n, method=2)).sum())
        want.reshape(-1)[i] = (f(hi) - f(lo)) / (2 * eps)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-8)
