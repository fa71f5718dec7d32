"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle,
the committed golden vectors and the reference's known answers.

Tolerances (per coefficient, relative to max(|expected|, largest |expected| of that level
and path)): 1e-10 in float64 and 1e-5 in float32."""
import numpy as np
import pytest
import torch

import cabi
from conftest import assert_grad_close, assert_grad_parity, assert_sig_close, brownian_paths
from oracle import oracle
from pysiglib_b200 import load_cusig

pytestmark = pytest.mark.gpu

RTOL = {np.float64: 1e-10, np.float32: 1e-5}


@pytest.fixture(params=[0, 1], ids=["auto", "generic"])
def policy(request):
    load_cusig.set_kernel_policy(request.param)
    yield request.param
    load_cusig.set_kernel_policy(0)


def run_forward(path, degree, **kw):
    code, out = cabi.signature_cuda(path, degree, pad=3, **kw)
    assert code == 0, load_cusig.last_error_message()
    assert np.all(out[-3:] == -1.0), "write past the end of the output"
    return out[:-3].reshape(path.shape[0], -1)


def run_backward(path, sig, derivs, degree, **kw):
    code, out = cabi.sig_backprop_cuda(path, sig, derivs, degree, pad=3, **kw)
    assert code == 0, load_cusig.last_error_message()
    assert np.all(out[-3:] == -1.0), "write past the end of the output"
    return out[:-3].reshape(path.shape)


# ---- golden vectors of the reference (tests/golden/reference_sig_vectors.npz) ----

@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 1e-4)])
def test_golden_sig(golden, policy, deg, dtype, tol):
    p3, p2 = golden["path"].astype(dtype), golden["path_dim2"].astype(dtype)
    np.testing.assert_allclose(run_forward(p3, deg), golden["sig__d%d" % deg], rtol=0, atol=tol)
    np.testing.assert_allclose(run_forward(p3, deg, time_aug=True), golden["sig_ta__d%d" % deg], rtol=0, atol=tol)
    np.testing.assert_allclose(run_forward(p2, deg, lead_lag=True), golden["sig_ll__d%d" % deg], rtol=0, atol=tol)
    np.testing.assert_allclose(run_forward(p2, deg, time_aug=True, lead_lag=True),
                               golden["sig_ta_ll__d%d" % deg], rtol=0, atol=tol)
    np.testing.assert_allclose(run_forward(p3, deg, horner=False), golden["sig__d%d" % deg], rtol=0, atol=tol)


@pytest.mark.parametrize("deg", range(1, 6))
def test_golden_sig_backprop(golden, policy, deg):
    path = golden["path"]
    derivs = np.ascontiguousarray(golden["sig_bp_derivs__d%d" % deg])
    sig = run_forward(path, deg, scalar_term=True)
    got = run_backward(path, sig, derivs, deg, scalar_term=True)
    np.testing.assert_allclose(got, golden["sig_bp_expected__d%d" % deg], rtol=0, atol=1e-5)


# ---- the reference's hand-computed vectors through the CUDA path ----

def test_known_answers(policy):
    path = np.array([0., 0., 1., .5, 4., 0., 0., 1.]).reshape(1, 4, 2)
    np.testing.assert_allclose(run_forward(path, 2, scalar_term=True)[0], [1., 0., 1., 0., 1., -1., .5], atol=1e-14)
    p = np.array([0, 5, 2, 4, 9], dtype=np.float32).reshape(1, 5, 1)
    ta = [1., 9., 4., 40.5, 15.5, 20.5, 8., 121.5, 37.5, 64.5, 24.5, 60., 13., 34.5, 10. + 2 / 3.]
    np.testing.assert_allclose(run_forward(p, 3, time_aug=True, end_time=4.0, scalar_term=True)[0], ta, rtol=2e-6)
    ll = [1., 9., 9., 40.5, 9., 72., 40.5, 121.5, 6.5, 68., -8.5, 290., 98., 275., 121.5]
    np.testing.assert_allclose(run_forward(p, 3, lead_lag=True, scalar_term=True)[0], ll, rtol=2e-6)
    # backward: ManualBatchTest of the reference's C++ unit tests
    path = np.array([0., 0., 1., 2., .5, 1., 0., 0., 3., 2., 5., 2., 0., 0., -1., 2., .5, -1.]).reshape(3, 3, 2)
    derivs = np.array([[1.] + list(range(1, 15)),
                       [1., 1., -2., 3., -4., 5., -6., 7., -8., 9., -10., 11., -12., 13., -14.], [1.] * 15])
    expect = [-19.625, -23.625, -1.25, .625, 20.875, 23., -162.5, -103.5, -81.0, 245.5, 243.5, -142.0,
              -.625, -.625, 0., 0., .625, .625]
    sig = run_forward(path, 3, scalar_term=True)
    np.testing.assert_allclose(run_backward(path, sig, derivs, 3, scalar_term=True).ravel(), expect, atol=1e-12)
    # flags: TimeAugLeadLagTest
    path = np.array([0., 2., 1.]).reshape(1, 3, 1)
    derivs = np.array([[1.] + list(range(1, 13))])
    sig = run_forward(path, 2, time_aug=True, lead_lag=True, end_time=4.0, scalar_term=True)
    np.testing.assert_allclose(sig[0], [1., 1., 1., 4., .5, -2., 4.5, 3., .5, 5.5, -.5, -1.5, 8.], atol=1e-13)
    got = run_backward(path, sig, derivs, 2, time_aug=True, lead_lag=True, end_time=4.0, scalar_term=True)
    np.testing.assert_allclose(got.ravel(), [-98., -6., 104.], atol=1e-12)


# ---- seeded random shapes against the oracle: every kernel family, both directions ----

SHAPES = [  # (B, L, d, N, time_aug, lead_lag)
    (3, 9, 2, 2, False, False), (5, 40, 2, 6, False, False), (2, 17, 2, 12, False, False),
    (4, 33, 3, 4, False, False), (3, 65, 3, 5, True, False), (2, 12, 4, 4, False, True),
    (6, 34, 5, 3, False, False), (2, 70, 5, 7, False, False), (3, 21, 6, 3, True, True),
    (2, 50, 8, 4, False, False), (2, 30, 10, 5, False, False), (3, 45, 16, 4, False, False),
    (2, 18, 16, 3, True, False), (2, 10, 16, 2, False, True), (3, 25, 7, 6, False, False),
    (2, 20, 11, 5, False, False), (2, 15, 40, 2, False, False), (70, 6, 3, 3, False, False),
    (1, 2, 4, 3, False, False), (2, 3, 2, 4, True, True), (2, 100, 1, 5, True, False),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "B%d_L%d_d%d_N%d_%d%d" % s)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_random_shapes_forward_backward(shape, dtype, scalar_term):
    B, L, d, N, ta, ll = shape
    path = brownian_paths(B * 7 + L + d + N, B, L, d, dtype) * 3.0
    kw = dict(time_aug=ta, lead_lag=ll, end_time=1.5)
    D = cabi.aug_dim(d, ta, ll)
    expect = oracle.sig(path, N, scalar_term=scalar_term, **kw)
    got = run_forward(path, N, scalar_term=scalar_term, **kw)
    assert_sig_close(got, expect, D, N, RTOL[dtype], scalar_term)

    rng = np.random.default_rng(B + N)
    seeds = np.ascontiguousarray(rng.normal(size=expect.shape).astype(dtype))
    want = oracle.sig_backprop(path, expect, seeds, N, **kw)
    p64 = path.astype(np.float64)
    truth = oracle.sig_backprop(p64, oracle.sig(p64, N, scalar_term=scalar_term, **kw), seeds.astype(np.float64), N, **kw)
    grad = run_backward(path, expect, seeds, N, scalar_term=scalar_term, **kw)
    assert_grad_parity(grad, want, truth, RTOL[dtype])


@pytest.mark.parametrize("shape", [(3, 20, 3, 4, False, False), (2, 30, 16, 4, False, False),
                                   (2, 25, 8, 4, True, False), (3, 15, 2, 6, False, True)],
                         ids=lambda s: "B%d_L%d_d%d_N%d_%d%d" % s)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_generic_kernels_match_oracle(shape, dtype):
    """Same shapes forced onto the shape-generic kernels."""
    B, L, d, N, ta, ll = shape
    load_cusig.set_kernel_policy(1)
    try:
        path = brownian_paths(L + d, B, L, d, dtype) * 2.0
        kw = dict(time_aug=ta, lead_lag=ll, end_time=0.7)
        expect = oracle.sig(path, N, **kw)
        got = run_forward(path, N, **kw)
        assert_sig_close(got, expect, cabi.aug_dim(d, ta, ll), N, RTOL[dtype])
        seeds = np.ones_like(expect)
        want = oracle.sig_backprop(path, expect, seeds, N, **kw)
        p64 = path.astype(np.float64)
        truth = oracle.sig_backprop(p64, oracle.sig(p64, N, **kw), seeds.astype(np.float64), N, **kw)
        grad = run_backward(path, expect, seeds, N, **kw)
        assert_grad_parity(grad, want, truth, RTOL[dtype])
    finally:
        load_cusig.set_kernel_policy(0)


@pytest.mark.parametrize("pref", [1, 2, 4], ids=["biggest", "smallest", "segmented"])
@pytest.mark.parametrize("shape", [(3, 41, 16, 4), (2, 37, 8, 4), (2, 50, 2, 12), (2, 33, 5, 7), (2, 21, 10, 5),
                                   (5, 29, 3, 4), (2, 40, 9, 4)], ids=lambda s: "B%d_L%d_d%d_N%d" % s)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_tile_variants_and_time_segmentation(pref, shape, dtype):
    """Every compiled tile variant of a shape (biggest / smallest register tile) and the
    time-segmented forward sweep (segments joined by Chen products) give the oracle's result."""
    B, L, d, N = shape
    load_cusig.set_tile_preference(pref)
    try:
        path = brownian_paths(B + L, B, L, d, dtype) * 2.0
        expect = oracle.sig(path, N)
        assert_sig_close(run_forward(path, N), expect, d, N, RTOL[dtype])
        assert_sig_close(run_forward(path, N, time_aug=True, scalar_term=True),
                         oracle.sig(path, N, time_aug=True, scalar_term=True), d + 1, N, RTOL[dtype], True)
        seeds = np.ascontiguousarray(np.random.default_rng(B).normal(size=expect.shape).astype(dtype))
        want = oracle.sig_backprop(path, expect, seeds, N)
        p64 = path.astype(np.float64)
        truth = oracle.sig_backprop(p64, oracle.sig(p64, N), seeds.astype(np.float64), N)
        assert_grad_parity(run_backward(path, expect, seeds, N), want, truth, RTOL[dtype])
        if d <= 5:  # flags through the same variants (lead-lag doubles the dimension)
            kw = dict(time_aug=True, lead_lag=(d <= 3), end_time=0.8)
            D = cabi.aug_dim(d, kw["time_aug"], kw["lead_lag"])
            n_small = min(N, 4)
            e2 = oracle.sig(path, n_small, **kw)
            assert_sig_close(run_forward(path, n_small, **kw), e2, D, n_small, RTOL[dtype])
            sd = np.ascontiguousarray(np.random.default_rng(L).normal(size=e2.shape).astype(dtype))
            w2 = oracle.sig_backprop(path, e2, sd, n_small, **kw)
            t2 = oracle.sig_backprop(p64, oracle.sig(p64, n_small, **kw), sd.astype(np.float64), n_small, **kw)
            assert_grad_parity(run_backward(path, e2, sd, n_small, **kw), w2, t2, RTOL[dtype])
    finally:
        load_cusig.set_tile_preference(0)


def test_float32_forward_tracks_reference_operation_order():
    """The kernels keep the reference's per-coefficient operation order (only nvcc's
    multiply-add contraction differs), so float32 forward results sit within a few ulp of
    the oracle's: 2e-6 relative to the level's largest coefficient."""
    path = brownian_paths(5, 4, 50, 5, np.float32)
    expect = oracle.sig(path, 4)
    for pol in (0, 1):
        load_cusig.set_kernel_policy(pol)
        try:
            got = run_forward(path, 4)
        finally:
            load_cusig.set_kernel_policy(0)
        assert_sig_close(got, expect, 5, 4, 2e-6)


# ---- edge cases the reference tests ----

def test_trivial_and_edge_cases(policy):
    one = np.zeros((2, 1, 3))
    assert run_forward(one, 3, scalar_term=True).tolist() == [[1.0] + [0.0] * 39] * 2
    assert run_forward(one, 3).tolist() == [[0.0] * 39] * 2
    p = brownian_paths(1, 3, 8, 3)
    assert run_forward(p, 0, scalar_term=True).tolist() == [[1.0]] * 3
    np.testing.assert_allclose(run_forward(p, 1), p[:, -1] - p[:, 0], atol=1e-15)
    q = brownian_paths(2, 3, 8, 1)
    np.testing.assert_allclose(run_forward(q, 5, scalar_term=True), oracle.sig(q, 5, scalar_term=True), rtol=1e-14)
    # backward trivial cases: length 1 and degree 0 give zeros, degree 1 only touches the end points
    s = run_forward(one, 2)
    assert not run_backward(one, s, np.ones_like(s), 2).any()
    s1 = run_forward(p, 1)
    g = run_backward(p, s1, np.ones_like(s1), 1)
    np.testing.assert_array_equal(g[:, 1:-1], 0.0)
    np.testing.assert_allclose(g[:, 0], -1.0)
    np.testing.assert_allclose(g[:, -1], 1.0)
    np.testing.assert_allclose(run_backward(q, run_forward(q, 4), np.ones((3, 4)), 4),
                               oracle.sig_backprop(q, oracle.sig(q, 4), np.ones((3, 4)), 4), rtol=1e-12)


def test_error_codes_and_messages():
    lib = load_cusig.library()
    p = np.zeros((1, 4, 2))
    out = np.zeros(64)
    dptr = ctypes_ptr = p.ctypes.data_as(__import__("ctypes").POINTER(__import__("ctypes").c_double))
    optr = out.ctypes.data_as(__import__("ctypes").POINTER(__import__("ctypes").c_double))
    # dimension 0 -> invalid argument (reference: siglib/cusig/cu_signature.cu:2610)
    assert lib.signature_cuda_d(dptr, optr, 1, 0, 4, 2, False, False, 1.0, True, False, None, 0, 0, 0) == 2
    assert "dimension 0" in load_cusig.last_error_message()
    # a successful call clears the message (reference: siglib/cusig_unit_testing/cu_test_signature.cpp:21-51)
    assert lib.signature_cuda_d(dptr, optr, 1, 2, 4, 2, False, False, 1.0, True, False, None, 0, 0, 0) == 0
    assert load_cusig.last_error_message() == ""
    # empty batch: success, nothing written
    out[:] = 7.0
    assert lib.signature_cuda_d(dptr, optr, 0, 2, 4, 2, False, False, 1.0, True, False, None, 0, 0, 0) == 0
    assert np.all(out == 7.0)
    # a correction whose length is not a prefix of levels 2..degree is rejected (cu_signature.cu:2028-2055)
    assert lib.signature_cuda_d(dptr, optr, 1, 2, 4, 2, False, False, 1.0, True, False, optr, 3, 0, 0) == 2
    assert "prefix" in load_cusig.last_error_message()
    assert lib.sig_backprop_cuda_d(dptr, optr, optr, optr, 1, 0, 4, 2, False, False, 1.0, False, None, 0, 0, 0) == 2
    # symbols outside the served path exist and fail cleanly
    assert lib.sig_kernel_cuda_d() == 10
    assert "not part of this build" in load_cusig.last_error_message()


def test_large_batch_crosses_grid_and_chunk_boundaries():
    """B = 70000 > 65535 (the reference's tests/test_cuda_grid_limits.py:27-35 case)."""
    path = brownian_paths(9, 70000, 4, 2, np.float32)
    got = run_forward(path, 2)
    np.testing.assert_allclose(got, oracle.sig(path, 2, n_threads=8), rtol=1e-5, atol=1e-6)


def test_wide_paths_like_the_reference_resource_limit_tests():
    """Shapes of the reference's tests/test_signature_cuda_shared_memory.py and
    tests/test_cuda_memory_fallbacks.py: very wide paths at low degree."""
    rng = np.random.default_rng(29)
    for dtype, tol in ((np.float32, 1e-5), (np.float64, 1e-10)):
        p = rng.normal(size=(16, 127, 98)).astype(dtype)
        np.testing.assert_allclose(run_forward(p, 1), oracle.sig(p, 1), rtol=tol, atol=tol)
        p = rng.normal(size=(1, 2, 350)).astype(dtype)
        s = run_forward(p, 2)
        assert_sig_close(s, oracle.sig(p, 2), 350, 2, tol)
        g = run_backward(p, s, np.ones_like(s), 2)
        np.testing.assert_allclose(g, oracle.sig_backprop(p, oracle.sig(p, 2), np.ones_like(s), 2), rtol=2e-4, atol=2e-4)
        p = rng.normal(size=(1, 127, 1000)).astype(dtype)
        s = run_forward(p, 1)
        np.testing.assert_allclose(s, p[:, -1] - p[:, 0], rtol=tol, atol=tol)
        g = run_backward(p, s, np.ones_like(s), 1)
        assert not g[:, 1:-1].any() and np.all(g[:, 0] == -1) and np.all(g[:, -1] == 1)
        # d = 100000, degree 1, weighted seeds; then lead-lag with d = 50000
        p = rng.normal(size=(1, 3, 100000)).astype(dtype)
        for scalar_term in (False, True):
            s = run_forward(p, 1, scalar_term=scalar_term)
            w = np.linspace(-0.25, 0.5, s.size).astype(dtype).reshape(s.shape)
            g = run_backward(p, s, w, 1, scalar_term=scalar_term)
            np.testing.assert_array_equal(g[0, 0], -w[0, -100000:])
            np.testing.assert_array_equal(g[0, 1], 0)
            np.testing.assert_array_equal(g[0, 2], w[0, -100000:])
        p = rng.normal(size=(1, 3, 50000)).astype(dtype)
        s = run_forward(p, 1, lead_lag=True)
        np.testing.assert_allclose(s, oracle.sig(p, 1, lead_lag=True), rtol=tol, atol=tol)
        g = run_backward(p, s, np.ones_like(s), 1, lead_lag=True)
        np.testing.assert_allclose(g, oracle.sig_backprop(p, oracle.sig(p, 1, lead_lag=True), np.ones_like(s), 1,
                                                          lead_lag=True), rtol=tol, atol=tol)


def test_concurrent_calls_from_two_host_threads():
    """The C ABI is callable from any host thread; device-pointer calls on different streams do not
    share scratch memory (stream-ordered pool), host-pointer calls serialise on the staging streams."""
    import threading
    import pysiglib_b200
    paths = [brownian_paths(40 + i, 64, 200, 8, np.float32) for i in range(2)]
    expect = [oracle.sig(p, 4, n_threads=4) for p in paths]
    results = [None, None, None, None]

    def device_worker(i):
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            t = torch.tensor(paths[i], device="cuda")
            for _ in range(5):
                s = pysiglib_b200.sig(t, 4)
                g = pysiglib_b200.sig_backprop(t, s, torch.ones_like(s), 4)
            st.synchronize()
        results[i] = (s.cpu().numpy(), g.cpu().numpy())

    def host_worker(i):
        for _ in range(3):
            results[2 + i] = pysiglib_b200.sig(paths[i], 4)

    threads = [threading.Thread(target=device_worker, args=(i,)) for i in range(2)] + \
              [threading.Thread(target=host_worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for i in range(2):
        assert_sig_close(results[i][0], expect[i], 8, 4, 1e-5)
        assert_sig_close(results[2 + i], expect[i], 8, 4, 1e-5)
        want = oracle.sig_backprop(paths[i], expect[i], np.ones_like(expect[i]), 4, n_threads=4)
        np.testing.assert_allclose(results[i][1], want, rtol=1e-3, atol=1e-4 * np.abs(want).max())


# ---- device pointers, streams, autograd ----

def test_device_pointers_and_python_api():
    import pysiglib_b200
    path = brownian_paths(3, 6, 40, 4)
    expect = oracle.sig(path, 4)
    t = torch.tensor(path, device="cuda")
    code, out = cabi.signature_cuda(t, 4)
    assert code == 0
    np.testing.assert_allclose(out.cpu().numpy().reshape(6, -1), expect, rtol=1e-12, atol=1e-15)
    s = pysiglib_b200.sig(t, 4)
    assert s.is_cuda and s.shape == (6, 340)
    np.testing.assert_allclose(s.cpu().numpy(), expect, rtol=1e-12, atol=1e-15)
    # numpy in -> numpy out, multi-dim batch, single path
    s_np = pysiglib_b200.sig(path.reshape(2, 3, 40, 4), 4)
    assert isinstance(s_np, np.ndarray) and s_np.shape == (2, 3, 340)
    np.testing.assert_allclose(s_np.reshape(6, -1), expect, rtol=1e-12, atol=1e-15)
    assert pysiglib_b200.sig(path[0], 4).shape == (340,)
    # non-default stream
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        s2 = pysiglib_b200.sig(t, 4)
    st.synchronize()
    assert torch.equal(s, s2)
    # backward through the python API, scalar-term layout accepted
    g = pysiglib_b200.sig_backprop(t, s, torch.ones_like(s), 4)
    want = oracle.sig_backprop(path, expect, np.ones_like(expect), 4)
    np.testing.assert_allclose(g.cpu().numpy(), want, rtol=1e-9, atol=1e-12)
    sfull = pysiglib_b200.sig(t, 4, scalar_term=True)
    g2 = pysiglib_b200.sig_backprop(t, sfull, torch.ones_like(sfull), 4)
    assert torch.allclose(g, g2)


def test_torch_api_autograd_matches_oracle_and_does_not_mutate_inputs():
    from pysiglib_b200 import torch_api
    path = brownian_paths(4, 5, 30, 3, np.float64)
    t = torch.tensor(path, device="cuda", requires_grad=True)
    before = t.detach().clone()
    s = torch_api.sig(t, 4, time_aug=True)
    s.sum().backward()   # grad_output is an expanded (stride-0) tensor
    assert torch.equal(t.detach(), before)
    expect = oracle.sig(path, 4, time_aug=True)
    want = oracle.sig_backprop(path, expect, np.ones_like(expect), 4, time_aug=True)
    np.testing.assert_allclose(t.grad.cpu().numpy(), want, rtol=1e-9, atol=1e-12)
    # non-contiguous input
    t2 = torch.tensor(np.ascontiguousarray(path.transpose(0, 2, 1)), device="cuda").transpose(1, 2).requires_grad_(True)
    torch_api.sig(t2, 4, time_aug=True).sum().backward()
    np.testing.assert_allclose(t2.grad.cpu().numpy(), want, rtol=1e-9, atol=1e-12)


def test_nonfinite_warning():
    import pysiglib_b200
    big = np.full((1, 3, 2), 1e200)
    big[0, 1] = -1e200
    with pytest.warns(RuntimeWarning, match="NaN or Inf"):
        pysiglib_b200.sig(torch.tensor(big, device="cuda"), 4)


def test_sharded_call_reports_a_failing_shard_without_hanging():
    """Host-side failure injection: a device ordinal that does not exist makes the whole call fail
    with 'invalid argument' and a message; nothing is launched and later calls work."""
    import pysiglib_b200
    path = brownian_paths(8, 10, 20, 3, np.float32)
    with pytest.raises(Exception, match="not available"):
        pysiglib_b200.sig_sharded(path, 3, devices=[0, 99])
    with pytest.raises(Exception, match="positive"):
        pysiglib_b200.sig_sharded(path, 3, devices=[])
    assert pysiglib_b200.sig_sharded(path, 3, devices=[0]).shape == (10, 39)


def test_sharded_single_device_matches_plain():
    import pysiglib_b200
    path = brownian_paths(8, 10, 20, 3, np.float32)
    a = pysiglib_b200.sig(path, 3)
    b = pysiglib_b200.sig_sharded(path, 3, devices=[0])
    np.testing.assert_array_equal(a, b)
    g = pysiglib_b200.sig_backprop_sharded(path, a, np.ones_like(a), 3, devices=[0])
    np.testing.assert_allclose(g, oracle.sig_backprop(path, oracle.sig(path, 3), np.ones_like(a), 3), rtol=1e-4,
                               atol=1e-5)


@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 1e-5)])
def test_sig_combine_matches_oracle_and_chen_identity(dtype, tol):
    import pysiglib_b200
    for (B, L, d, N) in ((5, 31, 3, 4), (3, 40, 8, 4), (2, 25, 2, 9), (4, 12, 1, 5)):
        p = brownian_paths(B + d, B, L, d, dtype) * 2.0
        m = L // 2
        for scalar_term in (False, True):
            a = pysiglib_b200.sig(p[:, :m + 1].copy(), N, scalar_term=scalar_term)
            b = pysiglib_b200.sig(p[:, m:].copy(), N, scalar_term=scalar_term)
            ab = pysiglib_b200.sig(p, N, scalar_term=scalar_term)
            got = pysiglib_b200.sig_combine(a, b, d, N)
            assert got.shape == ab.shape
            assert_sig_close(got, oracle.sig_combine(a, b, d, N), d, N, tol, scalar_term)
            assert_sig_close(got, ab, d, N, 20 * tol, scalar_term)
        ta, tb = torch.tensor(a, device="cuda"), torch.tensor(b, device="cuda")
        tg = pysiglib_b200.sig_combine(ta, tb, d, N)
        assert tg.is_cuda
        np.testing.assert_array_equal(tg.cpu().numpy(), got)
    with pytest.raises(ValueError):
        pysiglib_b200.sig_combine(np.zeros((2, 14)), np.zeros((2, 13)), 2, 3)


@pytest.mark.parametrize("deg", range(1, 6))
def test_golden_sig_combine_backprop(golden, deg):
    """The reference's iisignature vectors for sig_combine_backprop (tests/test_sig_combine_backprop.py),
    host arrays and device tensors, scalar-term layout."""
    import pysiglib_b200
    s1, s2 = golden["sig_comb_bp_sig1__d%d" % deg], golden["sig_comb_bp_sig2__d%d" % deg]
    derivs = golden["sig_comb_bp_derivs__d%d" % deg]
    d1, d2 = pysiglib_b200.sig_combine_backprop(derivs, s1, s2, 3, deg)
    np.testing.assert_allclose(d1[:, 1:], golden["sig_comb_bp_d1__d%d" % deg], rtol=0, atol=1e-5)
    np.testing.assert_allclose(d2[:, 1:], golden["sig_comb_bp_d2__d%d" % deg], rtol=0, atol=1e-5)
    assert not d1[:, 0].any() and not d2[:, 0].any()
    t1, t2 = pysiglib_b200.sig_combine_backprop(torch.tensor(derivs, device="cuda"), torch.tensor(s1, device="cuda"),
                                                torch.tensor(s2, device="cuda"), 3, deg)
    np.testing.assert_array_equal(t1.cpu().numpy(), d1)
    np.testing.assert_array_equal(t2.cpu().numpy(), d2)


@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 1e-5)])
def test_sig_combine_backprop_matches_oracle(dtype, tol):
    import pysiglib_b200
    rng = np.random.default_rng(12)
    for (B, d, N) in ((4, 3, 4), (2, 8, 4), (3, 2, 8), (2, 16, 3)):
        n = oracle.sig_length(d, N)
        a, b, g = (np.ascontiguousarray(rng.normal(size=(B, n)).astype(dtype)) for _ in range(3))
        d1, d2 = pysiglib_b200.sig_combine_backprop(g, a, b, d, N)
        w1, w2 = oracle.sig_combine_backprop(g, a, b, d, N)
        assert_sig_close(d1, w1, d, N, tol)
        assert_sig_close(d2, w2, d, N, tol)
