"""GPU parity of the operators either side of ``sig``: per-segment corrections, ``linear_sig``,
``sig_join`` (+ backward) and ``transform_path`` (+ backward), against the CPU oracle, the
reference's own known answers and, for corrections, the reference's CUDA kernels on the same GPU.

Tolerances: 1e-10 relative (float64) and 1e-5 relative (float32), per coefficient relative to the
largest magnitude of its level, as for the signature itself."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close, assert_sig_close
from oracle import oracle, refcuda

pytestmark = pytest.mark.gpu


def _rtol(dtype):
    return 1e-10 if dtype == np.float64 else 1e-5


def _paths(seed, shape, dtype, scale=0.3):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(shape).cumsum(-2) * scale).astype(dtype)


# ----- corrections ------------------------------------------------------------------------------

KNOWN = [  # path, degree, kwargs, correction, expected (reference tests/test_signature.py:126-188)
    (np.array([[0.0], [3.0]]), 4, {}, np.array([2.0]), [1.0, 3.0, 6.5, 10.5, 14.375]),
    (np.zeros((3, 1)), 3, {}, np.array([2.0]), [1.0, 0.0, 4.0, 0.0]),
    (np.zeros((2, 1)), 2, {"time_aug": True}, np.array([[2.0]]), [1.0, 0.0, 1.0, 2.0, 0.0, 0.0, 0.5]),
]


@pytest.mark.parametrize("case", range(len(KNOWN)))
@pytest.mark.parametrize("where", ["cuda", "numpy"])
def test_correction_known_answers(case, where):
    import pysiglib_b200
    path, degree, kw, corr, expected = KNOWN[case]
    if where == "cuda":
        out = pysiglib_b200.sig(torch.tensor(path, device="cuda"), degree, scalar_term=True,
                                correction=torch.tensor(corr, device="cuda"), **kw).cpu().numpy()
    else:
        out = pysiglib_b200.sig(path.copy(), degree, scalar_term=True, correction=corr.copy(), **kw)
    np.testing.assert_allclose(out, expected, rtol=1e-13, atol=1e-14)


def test_empty_correction_matches_default():
    import pysiglib_b200
    x = torch.tensor(_paths(0, (3, 20, 3), np.float64), device="cuda")
    a = pysiglib_b200.sig(x, 4)
    b = pysiglib_b200.sig(x, 4, correction=torch.empty((0,), dtype=x.dtype, device="cuda"))
    assert torch.equal(a, b)


CORR_CASES = [  # (B, L, d, N, levels of correction, time_aug, layout, dtype)
    (3, 12, 2, 3, 1, False, "constant", np.float64),
    (3, 12, 2, 4, 3, False, "shared", np.float64),
    (5, 9, 3, 4, 2, True, "full", np.float64),
    (2, 30, 1, 5, 4, False, "full", np.float64),
    (4, 17, 4, 3, 2, False, "full", np.float32),
    (2, 8, 2, 6, 2, True, "shared", np.float32),
    (300, 6, 3, 3, 1, False, "full", np.float32),
]


def _correction(seed, B, L, d, levels, layout, dtype):
    rng = np.random.default_rng(seed)
    clen = sum(d ** k for k in range(2, 2 + levels))
    shape = {"constant": (clen,), "shared": (L - 1, clen), "full": (B, L - 1, clen)}[layout]
    c = (rng.standard_normal(shape) * 0.2).astype(dtype)
    c[..., ::7] = 0  # exact zeros are skipped by the scatter (cu_signature.cu:2095-2097)
    return c


@pytest.mark.parametrize("case", CORR_CASES, ids=lambda c: "B%d_L%d_d%d_N%d_k%d_%s_%s_%s" % (c[:5] + (c[5], c[6], c[7].__name__)))
@pytest.mark.parametrize("scalar_term", [False, True])
def test_correction_forward_and_backward(case, scalar_term):
    import pysiglib_b200
    B, L, d, N, levels, ta, layout, dtype = case
    path = _paths(B + L + d, (B, L, d), dtype)
    corr = _correction(N + levels, B, L, d, levels, layout, dtype)
    kw = dict(time_aug=ta, end_time=0.7)
    D = d + (1 if ta else 0)
    want = oracle.sig(path, N, scalar_term=scalar_term, correction=corr, **kw)
    pt, ct = torch.tensor(path, device="cuda"), torch.tensor(corr, device="cuda")
    got = pysiglib_b200.sig(pt, N, scalar_term=scalar_term, correction=ct, **kw)
    off = 1 if scalar_term else 0
    assert_sig_close(got.cpu().numpy()[:, off:], want[:, off:], D, N, _rtol(dtype))
    if scalar_term:
        assert torch.all(got[:, 0] == 1)
    # host buffers take the staged route to the same kernels
    got_host = pysiglib_b200.sig(path, N, scalar_term=scalar_term, correction=corr, **kw)
    np.testing.assert_array_equal(got_host, got.cpu().numpy())

    seeds = np.random.default_rng(7).standard_normal(want.shape).astype(dtype)
    p64, c64 = path.astype(np.float64), corr.astype(np.float64)
    truth = oracle.sig_backprop(p64, oracle.sig(p64, N, scalar_term=scalar_term, correction=c64, **kw),
                                seeds.astype(np.float64), N, correction=c64, **kw)
    grad = pysiglib_b200.sig_backprop(pt, torch.tensor(want, device="cuda"), torch.tensor(seeds, device="cuda"), N,
                                      correction=ct, **kw)
    assert_grad_close(grad.cpu().numpy(), truth, 1e-9 if dtype == np.float64 else 2e-4)
    grad_host = pysiglib_b200.sig_backprop(path, want, seeds, N, correction=corr, **kw)
    assert_grad_close(grad_host, truth, 1e-9 if dtype == np.float64 else 2e-4)


@pytest.mark.skipif(not refcuda.available(), reason="reference CUDA library not built")
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_correction_matches_reference_cuda(dtype):
    import pysiglib_b200
    B, L, d, N = 6, 40, 3, 4
    path = torch.tensor(_paths(1, (B, L, d), dtype), device="cuda")
    corr = torch.tensor(_correction(2, B, L, d, 2, "full", dtype), device="cuda")
    ref = refcuda.sig(path, N, correction=corr)
    ours = pysiglib_b200.sig(path, N, correction=corr)
    assert_sig_close(ours.cpu().numpy(), ref.cpu().numpy(), d, N, _rtol(dtype))
    seeds = torch.randn(ref.shape, dtype=ref.dtype, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    ref_g = refcuda.sig_backprop(path, ref, seeds, N, correction=corr)
    our_g = pysiglib_b200.sig_backprop(path, ref, seeds, N, correction=corr)
    assert_grad_close(our_g.cpu().numpy(), ref_g.cpu().numpy().astype(np.float64), 1e-9 if dtype == np.float64 else 3e-4)


def test_correction_autograd():
    from pysiglib_b200 import torch_api
    path = torch.tensor(_paths(4, (3, 10, 2), np.float64), device="cuda", requires_grad=True)
    corr = torch.tensor(_correction(5, 3, 10, 2, 2, "shared", np.float64), device="cuda")
    out = torch_api.sig(path, 3, correction=corr)
    w = torch.randn(out.shape, dtype=out.dtype, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    (out * w).sum().backward()
    want = oracle.sig_backprop(path.detach().cpu().numpy(), out.detach().cpu().numpy(), w.cpu().numpy(), 3,
                               correction=corr.cpu().numpy())
    assert_grad_close(path.grad.cpu().numpy(), want, 1e-9)


def test_correction_errors():
    from pysiglib_b200 import load_cusig
    import cabi  # noqa: F401  (ensures the library is loaded the way the other ABI tests load it)
    import ctypes
    lib = load_cusig.library()
    x = torch.zeros((1, 3, 2), dtype=torch.float64, device="cuda")
    out = torch.zeros(6, dtype=torch.float64, device="cuda")
    c = torch.zeros(5, dtype=torch.float64, device="cuda")
    p = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_double))
    code = lib.signature_cuda_d(p(x), p(out), 1, 2, 3, 2, False, False, 1.0, True, False, p(c), 5, 0, 0)
    assert code == 2 and "prefix" in load_cusig.last_error_message()
    code = lib.signature_cuda_d(p(x), p(out), 1, 2, 3, 2, False, True, 1.0, True, False, p(c), 4, 0, 0)
    assert code == 2 and "lead_lag" in load_cusig.last_error_message()
    code = lib.signature_cuda_d(p(x), p(out), 1, 2, 3, 1, False, False, 1.0, True, False, p(c), 4, 0, 0)
    assert code == 2 and "degree < 2" in load_cusig.last_error_message()


# ----- linear_sig / sig_join ----------------------------------------------------------------------

JOIN_CASES = [(7, 1, 5), (5, 2, 6), (9, 3, 4), (4, 8, 3), (3, 16, 3), (600, 3, 3), (2, 5, 1), (2, 4, 0)]


@pytest.mark.parametrize("B,d,N", JOIN_CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_linear_sig(B, d, N, dtype, scalar_term):
    import pysiglib_b200
    v = np.random.default_rng(B + d + N).standard_normal((B, d)).astype(dtype)
    want = oracle.linear_sig(v, N, scalar_term=scalar_term)
    got = pysiglib_b200.linear_sig(torch.tensor(v, device="cuda"), d, N, scalar_term=scalar_term)
    assert got.shape == want.shape
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-14 if dtype == np.float64 else 1e-6, atol=0)
    got_host = pysiglib_b200.linear_sig(v, d, N, scalar_term=scalar_term)
    np.testing.assert_array_equal(got_host, got.cpu().numpy())


@pytest.mark.parametrize("B,d,N", JOIN_CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("prepend", [False, True])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_sig_join_and_backprop(B, d, N, dtype, prepend, scalar_term):
    import pysiglib_b200
    if N == 0 and not scalar_term:
        pytest.skip("empty signature")
    rng = np.random.default_rng(B * 100 + d * 10 + N)
    path = _paths(B + d, (B, 6, d), dtype)
    s = oracle.sig(path, N, scalar_term=scalar_term)
    v = (rng.standard_normal((B, d)) * 0.5).astype(dtype)
    want = oracle.sig_join(s, v, d, N, prepend=prepend)
    st, vt = torch.tensor(s, device="cuda"), torch.tensor(v, device="cuda")
    got = pysiglib_b200.sig_join(st, vt, d, N, prepend=prepend)
    off = 1 if scalar_term else 0
    if N > 0:
        assert_sig_close(got.cpu().numpy()[:, off:], want[:, off:], d, N, _rtol(dtype))
    if scalar_term:
        assert torch.all(got[:, 0] == 1)
    np.testing.assert_array_equal(pysiglib_b200.sig_join(s, v, d, N, prepend=prepend), got.cpu().numpy())

    g = rng.standard_normal(s.shape).astype(dtype)
    s64, v64, g64 = s.astype(np.float64), v.astype(np.float64), g.astype(np.float64)
    want_sig, want_disp = oracle.sig_join_backprop(g64, s64, v64, d, N, prepend=prepend)
    d_sig, d_disp = pysiglib_b200.sig_join_backprop(torch.tensor(g, device="cuda"), st, vt, d, N, prepend=prepend)
    tol = 1e-10 if dtype == np.float64 else 1e-4
    assert_grad_close(d_sig.cpu().numpy(), want_sig, tol)
    assert_grad_close(d_disp.cpu().numpy(), want_disp, tol)
    h_sig, h_disp = pysiglib_b200.sig_join_backprop(g, s, v, d, N, prepend=prepend)
    assert_grad_close(h_sig, want_sig, tol)
    assert_grad_close(h_disp, want_disp, tol)


def test_sig_join_extends_the_path():
    # reference tests/test_linear_and_branched_join.py:86-112: joining a displacement equals the
    # signature of the path with one more point
    import pysiglib_b200
    path = torch.tensor(_paths(9, (4, 30, 3), np.float64), device="cuda")
    v = torch.tensor(np.random.default_rng(1).standard_normal((4, 3)), device="cuda")
    s = pysiglib_b200.sig(path, 4)
    ext = torch.cat([path, path[:, -1:] + v[:, None]], dim=1).contiguous()
    assert_sig_close(pysiglib_b200.sig_join(s, v, 3, 4).cpu().numpy(), pysiglib_b200.sig(ext, 4).cpu().numpy(), 3, 4, 1e-10)
    pre = torch.cat([path[:, :1] - v[:, None], path], dim=1).contiguous()
    assert_sig_close(pysiglib_b200.sig_join(s, v, 3, 4, prepend=True).cpu().numpy(),
                     pysiglib_b200.sig(pre, 4).cpu().numpy(), 3, 4, 1e-10)


def test_sig_join_autograd_and_empty():
    from pysiglib_b200 import torch_api
    import pysiglib_b200
    s = torch.tensor(oracle.sig(_paths(3, (2, 5, 2), np.float64), 3), device="cuda", requires_grad=True)
    v = torch.tensor([[0.3, -0.2], [0.1, 0.4]], dtype=torch.float64, device="cuda", requires_grad=True)
    out = torch_api.sig_join(s, v, 2, 3)
    w = torch.arange(out.numel(), dtype=torch.float64, device="cuda").reshape(out.shape) / 10
    (out * w).sum().backward()
    ws, wv = oracle.sig_join_backprop(w.cpu().numpy(), s.detach().cpu().numpy(), v.detach().cpu().numpy(), 2, 3)
    assert_grad_close(s.grad.cpu().numpy(), ws, 1e-10)
    assert_grad_close(v.grad.cpu().numpy(), wv, 1e-10)
    empty = pysiglib_b200.sig_join(torch.zeros((0, 14), device="cuda"), torch.zeros((0, 2), device="cuda"), 2, 3)
    assert empty.shape == (0, 14)


# ----- transform_path -----------------------------------------------------------------------------

def _transform_ref(x, time_aug, lead_lag, end_time):
    """Plain-numpy statement of the transformed path (siglib/cusig/cu_path_transforms.cu:49-98)."""
    B, L, d = x.shape
    if lead_lag:
        out = np.empty((B, 2 * L - 1, 2 * d), dtype=x.dtype)
        out[:, 0::2, :d] = x
        out[:, 0::2, d:] = x
        out[:, 1::2, :d] = x[:, :-1]
        out[:, 1::2, d:] = x[:, 1:]
    else:
        out = x.copy()
    if time_aug:
        n = out.shape[1]
        scale = np.asarray(end_time, dtype=x.dtype) / np.asarray(n - 1, dtype=x.dtype)
        t = (np.arange(n).astype(x.dtype) * scale).astype(x.dtype)
        out = np.concatenate([out, np.broadcast_to(t[None, :, None], (B, n, 1))], axis=2)
    return out


@pytest.mark.parametrize("time_aug,lead_lag", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("shape", [(3, 7, 2), (1, 2, 5), (130, 33, 3)])
def test_transform_path_and_backprop(time_aug, lead_lag, dtype, shape):
    import pysiglib_b200
    x = np.random.default_rng(sum(shape)).standard_normal(shape).astype(dtype)
    want = _transform_ref(x, time_aug, lead_lag, 1.7)
    xt = torch.tensor(x, device="cuda")
    got = pysiglib_b200.transform_path(xt, time_aug=time_aug, lead_lag=lead_lag, end_time=1.7)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    np.testing.assert_array_equal(pysiglib_b200.transform_path(x, time_aug=time_aug, lead_lag=lead_lag, end_time=1.7), want)
    # the signature of the materialised path is the signature with the flags
    a = pysiglib_b200.sig(got, 3)
    b = pysiglib_b200.sig(xt, 3, time_aug=time_aug, lead_lag=lead_lag, end_time=1.7)
    assert_sig_close(a.cpu().numpy(), b.cpu().numpy(), want.shape[-1], 3, _rtol(dtype))
    # adjoint: <T x, g> = <x, T^* g> for the linear part of the map
    g = np.random.default_rng(1).standard_normal(want.shape).astype(dtype)
    back = pysiglib_b200.transform_path_backprop(torch.tensor(g, device="cuda"), time_aug=time_aug, lead_lag=lead_lag,
                                                 end_time=1.7).cpu().numpy()
    assert back.shape == x.shape
    lin = _transform_ref(x, False, lead_lag, 1.7).astype(np.float64)
    gl = g[..., :lin.shape[-1]].astype(np.float64)
    np.testing.assert_allclose((lin * gl).sum(), (x.astype(np.float64) * back).sum(), rtol=1e-5 if dtype == np.float32 else 1e-12)
    np.testing.assert_array_equal(
        pysiglib_b200.transform_path_backprop(g, time_aug=time_aug, lead_lag=lead_lag, end_time=1.7), back)


def test_transform_path_autograd():
    from pysiglib_b200 import torch_api
    x = torch.randn((2, 5, 2), dtype=torch.float64, device="cuda", requires_grad=True)
    y = torch_api.transform_path(x, time_aug=True, lead_lag=True)
    w = torch.randn(y.shape, dtype=y.dtype, device="cuda")
    (y * w).sum().backward()
    ref = torch.tensor(x.detach().cpu().numpy(), requires_grad=True)
    L = ref.shape[1]
    idx_even, idx_odd = torch.arange(L), torch.arange(L - 1)
    out = torch.zeros((2, 2 * L - 1, 4), dtype=torch.float64)
    out[:, 0::2, :2] = ref[:, idx_even]
    out[:, 0::2, 2:] = ref[:, idx_even]
    out[:, 1::2, :2] = ref[:, idx_odd]
    out[:, 1::2, 2:] = ref[:, idx_odd + 1]
    (out * w.cpu()[..., :4]).sum().backward()
    np.testing.assert_allclose(x.grad.cpu().numpy(), ref.grad.numpy(), rtol=1e-13)
