"""GPU parity of ``sig_coef`` / ``sig_coef_backprop`` against the CPU oracle and against the
entries of the full signature computed by the same library."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close
from oracle import oracle

pytestmark = pytest.mark.gpu

WORDS = [(0,), (1, 0), (2, 2, 1), (0, 1, 2, 0), (), (1, 1), (2, 0, 1, 1, 0, 2)]


def _paths(seed, shape, dtype):
    return (np.random.default_rng(seed).standard_normal(shape).cumsum(-2) * 0.3).astype(dtype)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("flags", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("prefixes", [False, True])
def test_forward_matches_oracle_and_full_signature(dtype, flags, prefixes):
    import pysiglib_b200
    ta, ll = flags
    path = _paths(1, (5, 40, 3), dtype)
    kw = dict(time_aug=ta, lead_lag=ll, end_time=1.5)
    want = oracle.sig_coef(path, WORDS, prefixes=prefixes, **kw)
    pt = torch.tensor(path, device="cuda")
    got = pysiglib_b200.sig_coef(pt, WORDS, prefixes=prefixes, **kw)
    assert got.shape == want.shape
    tol = dict(rtol=1e-10, atol=1e-12) if dtype == np.float64 else dict(rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(got.cpu().numpy(), want, **tol)
    np.testing.assert_array_equal(pysiglib_b200.sig_coef(path, WORDS, prefixes=prefixes, **kw), got.cpu().numpy())
    if not prefixes:
        words = [w for w in WORDS if w]
        full = pysiglib_b200.sig(pt, 6, **kw)
        picked = pysiglib_b200.extract_sig_coef(full, words, 3, time_aug=ta, lead_lag=ll)
        np.testing.assert_allclose(pysiglib_b200.sig_coef(pt, words, **kw).cpu().numpy(), picked.cpu().numpy(), **tol)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("flags", [(False, False), (True, True)])
def test_backward_matches_oracle(dtype, flags):
    import pysiglib_b200
    ta, ll = flags
    path = _paths(2, (4, 25, 3), dtype)
    kw = dict(time_aug=ta, lead_lag=ll, end_time=0.9)
    coefs = oracle.sig_coef(path, WORDS, prefixes=True, **kw)
    w = np.random.default_rng(3).standard_normal(coefs.shape).astype(dtype)
    p64 = path.astype(np.float64)
    want = oracle.sig_coef_backprop(p64, WORDS, oracle.sig_coef(p64, WORDS, prefixes=True, **kw), w.astype(np.float64), **kw)
    got = pysiglib_b200.sig_coef_backprop(torch.tensor(path, device="cuda"), WORDS, torch.tensor(coefs, device="cuda"),
                                          torch.tensor(w, device="cuda"), **kw)
    assert_grad_close(got.cpu().numpy(), want, 1e-9 if dtype == np.float64 else 3e-4)
    host = pysiglib_b200.sig_coef_backprop(path, WORDS, coefs, w, **kw)
    assert_grad_close(host, want, 1e-9 if dtype == np.float64 else 3e-4)


def test_autograd_and_edge_cases():
    from pysiglib_b200 import torch_api
    import pysiglib_b200
    path_np = _paths(4, (3, 12, 2), np.float64)
    path = torch.tensor(path_np, device="cuda", requires_grad=True)
    words = [(0, 1), (1, 1, 0)]
    out = torch_api.sig_coef(path, words, time_aug=True)
    assert out.shape == (3, 2)
    (out * torch.tensor([1.0, -2.0], device="cuda", dtype=torch.float64)).sum().backward()
    coefs = oracle.sig_coef(path_np, words, time_aug=True, prefixes=True)
    g = np.zeros_like(coefs)
    g[:, 1], g[:, 4] = 1.0, -2.0
    want = oracle.sig_coef_backprop(path_np, words, coefs, g, time_aug=True)
    assert_grad_close(path.grad.cpu().numpy(), want, 1e-9)
    # a single point, the empty word, many paths
    one = pysiglib_b200.sig_coef(torch.zeros((2, 1, 2), device="cuda"), [(0,), (), (1, 0)], prefixes=True)
    np.testing.assert_array_equal(one.cpu().numpy(), [[0, 1, 0, 0]] * 2)
    big = torch.tensor(_paths(5, (5000, 6, 2), np.float32), device="cuda")
    np.testing.assert_allclose(pysiglib_b200.sig_coef(big, (1, 0)).cpu().numpy(),
                               oracle.sig_coef(big.cpu().numpy(), (1, 0)), rtol=1e-4, atol=1e-6)


def test_errors():
    import ctypes
    from pysiglib_b200 import load_cusig
    lib = load_cusig.library()
    x = torch.zeros((1, 4, 2), dtype=torch.float64, device="cuda")
    out = torch.zeros(4, dtype=torch.float64, device="cuda")
    p = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_double))
    idx = (ctypes.c_uint64 * 2)(0, 5)
    deg = (ctypes.c_uint64 * 1)(2)
    assert lib.sig_coef_cuda_d(p(x), p(out), idx, 1, deg, 1, 2, 4, False) == 2
    assert "out of range" in load_cusig.last_error_message()
    deg = (ctypes.c_uint64 * 1)(40)
    assert lib.sig_coef_cuda_d(p(x), p(out), idx, 1, deg, 1, 2, 4, False) == 2
    assert "32 letters" in load_cusig.last_error_message()
