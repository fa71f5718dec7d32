"""Pins the CPU oracle: it must reproduce every golden vector and known answer the
reference's own tests hold for sig / sig_backprop, plus closed forms and an
independent autograd check.  Runs without a GPU."""
import numpy as np
import pytest
import torch

from oracle import oracle
from conftest import brownian_paths


# ---- the reference's iisignature fixture (its tests/test_signature.py:32-110) ----

@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 1e-4)])
@pytest.mark.parametrize("horner", [True, False])
def test_fixture_sig(golden, deg, dtype, tol, horner):
    path = golden["path"].astype(dtype)
    got = oracle.sig(path, deg, horner=horner)
    np.testing.assert_allclose(got, golden["sig__d%d" % deg], rtol=0, atol=tol)


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 1e-4)])
def test_fixture_sig_flags(golden, deg, dtype, tol):
    p3 = golden["path"].astype(dtype)
    p2 = golden["path_dim2"].astype(dtype)
    np.testing.assert_allclose(oracle.sig(p3, deg, time_aug=True), golden["sig_ta__d%d" % deg], rtol=0, atol=tol)
    np.testing.assert_allclose(oracle.sig(p2, deg, lead_lag=True), golden["sig_ll__d%d" % deg], rtol=0, atol=tol)
    np.testing.assert_allclose(oracle.sig(p2, deg, time_aug=True, lead_lag=True),
                               golden["sig_ta_ll__d%d" % deg], rtol=0, atol=tol)


@pytest.mark.parametrize("deg", range(1, 6))
def test_fixture_sig_backprop(golden, deg):
    # reference tests/test_sig_backprop.py:69-98: derivs carry the scalar slot, expected is float32
    path = golden["path"]
    derivs = golden["sig_bp_derivs__d%d" % deg]
    sig = oracle.sig(path, deg, scalar_term=True)
    got = oracle.sig_backprop(path, sig, derivs, deg)
    np.testing.assert_allclose(got, golden["sig_bp_expected__d%d" % deg], rtol=0, atol=1e-5)
    # scalar-free format gives the same answer
    got2 = oracle.sig_backprop(path, sig[:, 1:], derivs[:, 1:], deg)
    np.testing.assert_allclose(got2, got, rtol=0, atol=1e-13)


# ---- hand-computed vectors (reference siglib/cpsig_unit_testing/cp_test_signature.cpp) ----

def test_kat_trivial_cases():  # :140-160
    assert oracle.sig(np.zeros((1, 0, 1)), 0, scalar_term=True).tolist() == [[1.0]]
    assert oracle.sig(np.zeros((1, 1, 1)), 0, scalar_term=True).tolist() == [[1.0]]
    assert oracle.sig(np.zeros((1, 1, 1)), 1, scalar_term=True).tolist() == [[1.0, 0.0]]
    assert oracle.sig(np.array([[[0.0], [1.0]]]), 1, scalar_term=True).tolist() == [[1.0, 1.0]]


@pytest.mark.parametrize("pts", [[0., 0., .5, .5, 1., 1.], [0., 0., .25, .25, .75, .75, 1., 1.]])
def test_kat_linear_path(pts):  # :162-190
    path = np.array(pts).reshape(-1, 2)
    expect = [1.] + [1.] * 2 + [.5] * 4 + [1 / 6.] * 8
    np.testing.assert_allclose(oracle.sig(path, 3, scalar_term=True), expect, atol=1e-15)


def test_kat_manual_sig():  # :191-197
    path = np.array([0., 0., 1., .5, 4., 0., 0., 1.]).reshape(4, 2)
    np.testing.assert_allclose(oracle.sig(path, 2, scalar_term=True), [1., 0., 1., 0., 1., -1., .5], atol=1e-15)


def test_kat_manual_sig2_f32():  # :199-217
    path = np.array([9, 5, 8, 5, 3, 0, 0, 2, 6, 4, 0, 2], dtype=np.float32).reshape(4, 3)
    t = 1 / 3.
    expect = [1., -5., -5., -6., 12.5, 24.5, 5., .5, 12.5, 9., 25., 21., 18., -20.5 - t, -77.5 - t, 11.,
              33. + 1 / 6., -45.5 - t, -42. - t, -47., 5. + 2 * t, -18., -17.5 - t, -30.5 - t, 11. + 2 * t,
              14. + 1 / 6., -20.5 - t, -19., -14. - t, -7., -16. - 2 * t, -39., -110. - t, 6., -t, -49.,
              -20. - 2 * t, -78., -52. - 2 * t, -36.]
    np.testing.assert_allclose(oracle.sig(path, 3, scalar_term=True), expect, rtol=2e-6, atol=1e-5)


def test_kat_batch_and_degree1():  # :219-247
    path = np.array([0., 0., .25, .25, .5, .5, 1., 1., 0., 0., .4, .4, .6, .6, 1., 1.,
                     0., 0., 1., .5, 4., 0., 0., 1.]).reshape(3, 4, 2)
    e2 = np.array([[1., 1., 1., .5, .5, .5, .5]] * 2 + [[1., 0., 1., 0., 1., -1., .5]])
    for nt in (1, 3):
        np.testing.assert_allclose(oracle.sig(path, 2, scalar_term=True, n_threads=nt), e2, atol=1e-15)
    np.testing.assert_allclose(oracle.sig(path, 1, scalar_term=True), [[1, 1, 1], [1, 1, 1], [1, 0, 1]], atol=1e-15)


def test_kat_time_aug_and_lead_lag_f32():  # :249-265
    path = np.array([0, 5, 2, 4, 9], dtype=np.float32).reshape(5, 1)
    ta = [1., 9., 4., 40.5, 15.5, 20.5, 8., 121.5, 37.5, 64.5, 24.5, 60., 13., 34.5, 10. + 2 / 3.]
    np.testing.assert_allclose(oracle.sig(path, 3, time_aug=True, end_time=4.0, scalar_term=True), ta, rtol=2e-6)
    ll = [1., 9., 9., 40.5, 9., 72., 40.5, 121.5, 6.5, 68., -8.5, 290., 98., 275., 121.5]
    np.testing.assert_allclose(oracle.sig(path, 3, lead_lag=True, scalar_term=True), ll, rtol=2e-6)


BP_CASES = [  # (path, d, L, N, derivs, sig, expected, time_aug, lead_lag, end_time)   :277-405
    ([0., 0., 1., 1.], 2, 2, 2, [1.] * 7, [1., 1., 1., .5, .5, .5, .5], [-3., -3., 3., 3.], False, False, 1.),
    ([0., 0., 1., 2., .5, 1.], 2, 3, 2, [1., 1., 2., 3., 4., 5., 6.], [1., .5, 1., .125, .25, .25, .5],
     [-7.5, -10., -.5, .25, 8., 9.75], False, False, 1.),
    ([0., 0., 1., 2., .5, 1.], 2, 3, 3, [1.] + list(range(1, 15)),
     [1., .5, 1., .125, .25, .25, .5, 1 / 48., 1 / 24., 1 / 24., 1 / 12., 1 / 24., 1 / 12., 1 / 12., 1 / 6.],
     [-19.625, -23.625, -1.25, .625, 20.875, 23.], False, False, 1.),
    ([0., 2., 1.], 1, 3, 3, [1.] + list(range(1, 15)),
     [1., 1., 2., .5, 2.5, -.5, 2., 1 / 6., 1.5 + 1 / 3., -1 - 1 / 6., 2 + 1 / 6., 1 / 3., 2 / 3., -.5 - 1 / 3., 1 + 1 / 3.],
     [-54., -4.5, 58.5], True, False, 2.),
    ([0., 2., 1.], 1, 3, 3, [1.] + list(range(1, 15)),
     [1., 1., 1., .5, -2., 3., .5, 1 / 6., -2., 2., 1., .5, -4., 3.5, 1 / 6.],
     [-76., 5.5, 70.5], False, True, 1.),
    ([0., 2., 1.], 1, 3, 2, [1.] + list(range(1, 13)),
     [1., 1., 1., 4., .5, -2., 4.5, 3., .5, 5.5, -.5, -1.5, 8.],
     [-98., -6., 104.], True, True, 4.),
]


@pytest.mark.parametrize("case", BP_CASES)
def test_kat_backprop(case):
    pts, d, L, N, derivs, sig, expect, ta, ll, end_time = case
    path = np.array(pts).reshape(L, d)
    sig = np.array(sig, dtype=np.float64)
    # the hand-written signature in the reference test is the true one
    np.testing.assert_allclose(oracle.sig(path, N, time_aug=ta, lead_lag=ll, end_time=end_time, scalar_term=True),
                               sig, atol=1e-12)
    got = oracle.sig_backprop(path, sig, np.array(derivs, dtype=np.float64), N, time_aug=ta, lead_lag=ll,
                              end_time=end_time)
    np.testing.assert_allclose(got.ravel(), expect, atol=1e-12)


def test_kat_backprop_batch():  # ManualBatchTest :327-337
    path = np.array([0., 0., 1., 2., .5, 1., 0., 0., 3., 2., 5., 2., 0., 0., -1., 2., .5, -1.]).reshape(3, 3, 2)
    derivs = np.array([[1.] + list(range(1, 15)),
                       [1., 1., -2., 3., -4., 5., -6., 7., -8., 9., -10., 11., -12., 13., -14.],
                       [1.] * 15])
    expect = [-19.625, -23.625, -1.25, .625, 20.875, 23., -162.5, -103.5, -81.0, 245.5, 243.5, -142.0,
              -.625, -.625, 0., 0., .625, .625]
    sig = oracle.sig(path, 3, scalar_term=True)
    for nt in (1, 2):
        got = oracle.sig_backprop(path, sig, derivs, 3, n_threads=nt)
        np.testing.assert_allclose(got.ravel(), expect, atol=1e-12)


# ---- closed forms and independent checks ----

def test_linear_path_closed_form_high_degree():  # reference tests/test_cuda_horner.py:100-112
    direction = np.array([0.3, -0.2])
    path = np.linspace(0, 1, 9)[:, None] * direction[None]
    sig = oracle.sig(path, 14)
    start, level, fact = 0, np.ones(1), 1.0
    for k in range(1, 15):
        level = np.kron(level, direction)
        fact *= k
        np.testing.assert_allclose(sig[start:start + 2 ** k], level / fact, rtol=1e-9, atol=1e-18)
        start += 2 ** k


def test_dim1_closed_form():  # reference tests/test_signature.py:223-236
    path = np.array([[0.5], [2.0], [-1.0], [3.5]])
    sig = oracle.sig(path, 6, scalar_term=True)
    dx, fact = 3.0, 1.0
    for k in range(7):
        fact *= max(k, 1)
        np.testing.assert_allclose(sig[k], dx ** k / fact, rtol=1e-14)


def test_chen_identity():
    p = brownian_paths(7, 1, 17, 3)[0]
    a, b, ab = (oracle.sig(x, 4, scalar_term=True) for x in (p[:9], p[8:], p))
    # tensor product truncated at degree 4
    d, off = 3, [0, 1, 4, 13, 40, 121]
    prod = np.zeros_like(ab)
    for k in range(5):
        for i in range(k + 1):
            prod[off[k]:off[k + 1]] += np.kron(a[off[i]:off[i + 1]], b[off[k - i]:off[k - i + 1]])
    np.testing.assert_allclose(prod, ab, rtol=1e-12, atol=1e-15)


def _torch_sig(path, degree):
    """Independent reference: Chen products of segment exponentials in torch (autograd-able)."""
    d = path.shape[-1]
    levels = [torch.ones(1, dtype=path.dtype)] + [torch.zeros(d ** k, dtype=path.dtype) for k in range(1, degree + 1)]
    for t in range(path.shape[0] - 1):
        z = path[t + 1] - path[t]
        e = [torch.ones(1, dtype=path.dtype)]
        for k in range(1, degree + 1):
            e.append(torch.kron(e[-1], z) / k)
        levels = [sum(torch.kron(levels[i], e[k - i]) for i in range(k + 1)) for k in range(degree + 1)]
    return torch.cat(levels[1:])


@pytest.mark.parametrize("d,N,L", [(2, 4, 6), (3, 3, 5), (4, 2, 7), (1, 3, 4)])
def test_backprop_matches_independent_autograd(d, N, L):
    rng = np.random.default_rng(d * 100 + N)
    path = rng.normal(size=(L, d))
    seeds = rng.normal(size=oracle.sig_length(d, N))
    tp = torch.tensor(path, requires_grad=True)
    ts = _torch_sig(tp, N)
    (ts * torch.tensor(seeds)).sum().backward()
    sig = oracle.sig(path, N)
    np.testing.assert_allclose(sig, ts.detach().numpy(), rtol=1e-12, atol=1e-14)
    got = oracle.sig_backprop(path, sig, seeds, N)
    np.testing.assert_allclose(got, tp.grad.numpy(), rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("ta,ll", [(True, False), (False, True), (True, True)])
def test_backprop_flags_match_explicit_transform(ta, ll):
    # reference tests/test_sig_backprop.py:100-199: flags == autograd through the explicit transform
    rng = np.random.default_rng(11)
    L, d, N, end_time = 5, 2, 3, 1.7
    path = rng.normal(size=(L, d))
    tp = torch.tensor(path, requires_grad=True)
    x = tp
    if ll:
        rep = torch.repeat_interleave(x, 2, dim=0)
        x = torch.cat([rep[:-1], rep[1:]], dim=1)  # [lag, lead]
    if ta:
        t = torch.linspace(0, end_time, x.shape[0], dtype=x.dtype)[:, None]
        x = torch.cat([x, t], dim=1)
    dim = x.shape[1]
    seeds = rng.normal(size=oracle.sig_length(dim, N))
    ts = _torch_sig(x, N)
    (ts * torch.tensor(seeds)).sum().backward()
    sig = oracle.sig(path, N, time_aug=ta, lead_lag=ll, end_time=end_time)
    np.testing.assert_allclose(sig, ts.detach().numpy(), rtol=1e-11, atol=1e-13)
    got = oracle.sig_backprop(path, sig, seeds, N, time_aug=ta, lead_lag=ll, end_time=end_time)
    np.testing.assert_allclose(got, tp.grad.numpy(), rtol=1e-9, atol=1e-11)


def test_scalar_term_consistency_and_threads():  # reference tests/test_scalar_term.py:45-64
    p = brownian_paths(3, 5, 12, 3)
    a = oracle.sig(p, 4, scalar_term=True, n_threads=3)
    b = oracle.sig(p, 4, scalar_term=False)
    assert np.all(a[:, 0] == 1.0)
    np.testing.assert_array_equal(a[:, 1:], b)


def test_sig_combine_is_chen_identity():  # reference tests: sig(x1 * x2) == sig_combine(sig(x1), sig(x2))
    p = brownian_paths(9, 4, 21, 3)
    for scalar_term in (False, True):
        a = oracle.sig(p[:, :11], 4, scalar_term=scalar_term)
        b = oracle.sig(p[:, 10:], 4, scalar_term=scalar_term)
        ab = oracle.sig(p, 4, scalar_term=scalar_term)
        np.testing.assert_allclose(oracle.sig_combine(a, b, 3, 4), ab, rtol=1e-12, atol=1e-15)
    # hand-computed: level 2 of the product is a2 + b2 + a1 (x) b1
    s1 = np.array([1., 1., 1., .5, .5, .5, .5])
    s2 = np.array([1., 0., 1., 0., 1., -1., .5])
    np.testing.assert_allclose(oracle.sig_combine(s1, s2, 2, 2), [1., 1., 2., .5, 2.5, -.5, 2.], atol=1e-15)


@pytest.mark.parametrize("deg", range(1, 6))
def test_fixture_sig_combine_backprop(golden, deg):
    # reference tests/test_sig_combine_backprop.py:28-67 (dimension 3, inputs carry the scalar slot)
    s1, s2 = golden["sig_comb_bp_sig1__d%d" % deg], golden["sig_comb_bp_sig2__d%d" % deg]
    derivs = golden["sig_comb_bp_derivs__d%d" % deg]
    d1, d2 = oracle.sig_combine_backprop(derivs, s1, s2, 3, deg)
    np.testing.assert_allclose(d1[:, 1:], golden["sig_comb_bp_d1__d%d" % deg], rtol=0, atol=1e-5)
    np.testing.assert_allclose(d2[:, 1:], golden["sig_comb_bp_d2__d%d" % deg], rtol=0, atol=1e-5)
    assert not d1[:, 0].any() and not d2[:, 0].any()


def test_sig_combine_backprop_matches_autograd():
    rng = np.random.default_rng(4)
    d, N = 3, 3
    n = oracle.sig_length(d, N)
    a, b, g = rng.normal(size=n), rng.normal(size=n), rng.normal(size=n)
    ta, tb = torch.tensor(a, requires_grad=True), torch.tensor(b, requires_grad=True)
    off = [0, 3, 12, 39]
    la = [torch.ones(1, dtype=torch.float64)] + [ta[off[k]:off[k + 1]] for k in range(N)]
    lb = [torch.ones(1, dtype=torch.float64)] + [tb[off[k]:off[k + 1]] for k in range(N)]
    prod = torch.cat([sum(torch.kron(la[i], lb[k - i]) for i in range(k + 1)) for k in range(1, N + 1)])
    np.testing.assert_allclose(oracle.sig_combine(a, b, d, N), prod.detach().numpy(), rtol=1e-13)
    (prod * torch.tensor(g)).sum().backward()
    d1, d2 = oracle.sig_combine_backprop(g, a, b, d, N)
    np.testing.assert_allclose(d1, ta.grad.numpy(), rtol=1e-12, atol=1e-14)
    np.testing.assert_allclose(d2, tb.grad.numpy(), rtol=1e-12, atol=1e-14)
