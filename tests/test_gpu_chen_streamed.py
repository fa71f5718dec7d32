"""The one-CTA-per-signature Chen kernels (sig_chen.cu) only run for batches of at least one
signature per SM, so these cases use batches of 150 and more: sig_combine / sig_join and both backward
passes against the CPU oracle, over the vector widths (dimension a multiple of 4, of 2, odd), both
layouts (the scalar term shifts the alignment of every level), both dtypes, and shapes whose words per
prefix are below, equal to and above one warp's worth.  The launch counter shows that the streamed
kernels, not the per-coefficient ones, produced the result."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close, assert_sig_close
from oracle import oracle

pytestmark = pytest.mark.gpu

CASES = [(150, 4, 4), (160, 3, 5), (149, 6, 3), (200, 16, 3), (150, 2, 7), (170, 5, 2), (300, 8, 4), (150, 7, 3),
         (150, 32, 2), (150, 12, 3),
         # several iterations per level and suffix blocks longer than one iteration (register sums that
         # are flushed when the block offset changes), many splits, and degrees beyond the register path
         (150, 4, 7), (150, 8, 5), (148, 16, 4), (150, 2, 8), (150, 2, 10), (150, 64, 2), (150, 4, 2)]


def _adjoints_fit_shared_memory(d, N, dtype):
    """The adjoint kernel keeps four copies of the levels below N in shared memory (160 KB at most);
    larger signatures take the per-coefficient kernels, which is allowed."""
    low = sum(d ** k for k in range(N))
    return (4 * ((low + 6) & ~3) + 2 * ((d + 3) & ~3)) * np.dtype(dtype).itemsize <= 160 * 1024


def _signatures(seed, B, d, N, dtype, scalar_term):
    """Random signature-like arrays with levels that decay like a real signature's."""
    rng = np.random.default_rng(seed)
    n = oracle.sig_length(d, N)
    s = rng.standard_normal((B, n))
    pos = 0
    for k in range(1, N + 1):
        s[:, pos:pos + d ** k] *= 0.7 ** k / np.sqrt(float(d) ** (k - 1))
        pos += d ** k
    if scalar_term:
        s = np.concatenate([np.ones((B, 1)), s], axis=1)
    return np.ascontiguousarray(s.astype(dtype))


@pytest.mark.parametrize("B,d,N", CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_streamed_sig_combine_and_backprop(B, d, N, dtype, scalar_term):
    import pysiglib_b200
    from pysiglib_b200 import load_cusig
    a = _signatures(1, B, d, N, dtype, scalar_term)
    b = _signatures(2, B, d, N, dtype, scalar_term)
    g = _signatures(3, B, d, N, dtype, scalar_term)
    ta, tb, tg = (torch.tensor(x, device="cuda") for x in (a, b, g))
    tol = 1e-12 if dtype == np.float64 else 2e-6
    before = load_cusig.launch_count()
    got = pysiglib_b200.sig_combine(ta, tb, d, N)
    assert load_cusig.launch_count() - before == 1           # one kernel for the whole product
    assert_sig_close(got.cpu().numpy(), oracle.sig_combine(a, b, d, N), d, N, tol, scalar_term)

    before = load_cusig.launch_count()
    d1, d2 = pysiglib_b200.sig_combine_backprop(tg, ta, tb, d, N)
    if _adjoints_fit_shared_memory(d, N, dtype):
        assert load_cusig.launch_count() - before == 1       # both adjoints from one pass
    w1, w2 = oracle.sig_combine_backprop(g.astype(np.float64), a.astype(np.float64), b.astype(np.float64), d, N)
    gtol = 1e-11 if dtype == np.float64 else 2e-5
    assert_sig_close(d1.cpu().numpy(), w1, d, N, gtol, scalar_term, what="d sig1")
    assert_sig_close(d2.cpu().numpy(), w2, d, N, gtol, scalar_term, what="d sig2")
    if scalar_term:
        assert not d1[:, 0].any() and not d2[:, 0].any()


@pytest.mark.parametrize("B,d,N", CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("prepend", [False, True])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_streamed_sig_join_and_backprop(B, d, N, dtype, prepend, scalar_term):
    import pysiglib_b200
    from pysiglib_b200 import load_cusig
    s = _signatures(4, B, d, N, dtype, scalar_term)
    g = _signatures(5, B, d, N, dtype, scalar_term)
    v = (np.random.default_rng(6).standard_normal((B, d)) * 0.5).astype(dtype)
    ts, tg, tv = (torch.tensor(x, device="cuda") for x in (s, g, v))
    tol = 1e-12 if dtype == np.float64 else 2e-6
    before = load_cusig.launch_count()
    got = pysiglib_b200.sig_join(ts, tv, d, N, prepend=prepend)
    assert load_cusig.launch_count() - before == 1
    assert_sig_close(got.cpu().numpy(), oracle.sig_join(s, v, d, N, prepend=prepend), d, N, tol, scalar_term)

    before = load_cusig.launch_count()
    d_sig, d_disp = pysiglib_b200.sig_join_backprop(tg, ts, tv, d, N, prepend=prepend)
    if _adjoints_fit_shared_memory(d, N, dtype):
        assert load_cusig.launch_count() - before == 1
    want_sig, want_disp = oracle.sig_join_backprop(g.astype(np.float64), s.astype(np.float64), v.astype(np.float64), d, N,
                                                   prepend=prepend)
    gtol = 1e-11 if dtype == np.float64 else 2e-5
    assert_sig_close(d_sig.cpu().numpy(), want_sig, d, N, gtol, scalar_term, what="d sig")
    assert_grad_close(d_disp.cpu().numpy(), want_disp, gtol, what="d displacement")
    if scalar_term:
        assert not d_sig[:, 0].any()


def test_streamed_and_per_coefficient_kernels_agree():
    """The same signatures once as a small batch (per-coefficient kernels) and once inside a big one."""
    import pysiglib_b200
    d, N = 4, 5
    a = torch.tensor(_signatures(7, 200, d, N, np.float64, False), device="cuda")
    b = torch.tensor(_signatures(8, 200, d, N, np.float64, False), device="cuda")
    g = torch.tensor(_signatures(9, 200, d, N, np.float64, False), device="cuda")
    big = pysiglib_b200.sig_combine(a, b, d, N)
    small = pysiglib_b200.sig_combine(a[:5].contiguous(), b[:5].contiguous(), d, N)
    torch.testing.assert_close(big[:5], small, rtol=1e-13, atol=1e-15)
    big1, big2 = pysiglib_b200.sig_combine_backprop(g, a, b, d, N)
    s1, s2 = pysiglib_b200.sig_combine_backprop(g[:5].contiguous(), a[:5].contiguous(), b[:5].contiguous(), d, N)
    torch.testing.assert_close(big1[:5], s1, rtol=1e-12, atol=1e-14)
    torch.testing.assert_close(big2[:5], s2, rtol=1e-12, atol=1e-14)
