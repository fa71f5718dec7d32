"""GPU parity of ``sig_to_log_sig`` (+ backward) and ``log_sig`` for methods 0 and 1, against the
CPU oracle (``oracle/sig_oracle_log.h``).  Tolerances: 1e-10 relative (float64), 1e-5 relative
(float32), per coefficient relative to the largest magnitude of its level."""
import numpy as np
import pytest
import torch

from conftest import assert_grad_close, assert_sig_close, brownian_paths
from oracle import oracle

pytestmark = pytest.mark.gpu

CASES = [(5, 1, 6), (7, 2, 1), (6, 2, 7), (4, 3, 4), (3, 5, 3), (2, 8, 3), (70000, 2, 3), (2, 16, 3)]


def _assert_log_close(got, want, sig, d, N, rtol):
    """Per coefficient, relative to the largest term the series log(1+x) = x - x^2/2 + .. sums at
    that level: the level of the signature itself and the k-th power of its first level over k
    (the logarithm is what is left after these cancel)."""
    start = 0
    first = np.abs(sig[:, :d]).max(axis=1, keepdims=True).astype(np.float64)
    for k in range(1, N + 1):
        sl = slice(start, start + d ** k)
        start += d ** k
        floor = np.maximum(np.abs(want[:, sl]).max(axis=1, keepdims=True), np.abs(sig[:, sl]).max(axis=1, keepdims=True))
        floor = np.maximum(floor, first ** k / k)
        err = np.abs(got[:, sl].astype(np.float64) - want[:, sl]) / np.maximum(np.maximum(np.abs(want[:, sl]), floor), 1e-300)
        assert err.max() <= rtol, "log level %d: max scaled rel err %.3e > %.1e" % (k, err.max(), rtol)


def _sigs(seed, B, d, N, dtype, scalar_term):
    rng = np.random.default_rng(seed)
    path = (rng.standard_normal((B, 9, d)).cumsum(1) * 0.4).astype(dtype)
    return oracle.sig(path, N, scalar_term=scalar_term)


@pytest.mark.parametrize("B,d,N", CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_expanded_log_and_backprop(B, d, N, dtype, scalar_term):
    import pysiglib_b200
    s = _sigs(B + d + N, B, d, N, dtype, scalar_term)
    want = oracle.sig_to_log_sig(s, d, N, method=0)
    st = torch.tensor(s, device="cuda")
    got = pysiglib_b200.sig_to_log_sig(st, d, N, method=0)
    assert got.shape == st.shape
    off = 1 if scalar_term else 0
    rtol = 1e-10 if dtype == np.float64 else 1e-5
    _assert_log_close(got.cpu().numpy()[:, off:], want[:, off:], s[:, off:], d, N, rtol)
    if scalar_term:
        assert torch.all(got[:, 0] == 0)
    if B <= 64:
        np.testing.assert_array_equal(pysiglib_b200.sig_to_log_sig(s, d, N, method=0), got.cpu().numpy())

    w = np.random.default_rng(1).standard_normal(s.shape).astype(dtype)
    want_g = oracle.sig_to_log_sig_backprop(s.astype(np.float64), w.astype(np.float64), d, N, method=0)
    got_g = pysiglib_b200.sig_to_log_sig_backprop(st, torch.tensor(w, device="cuda"), d, N, method=0)
    assert_grad_close(got_g.cpu().numpy()[:, None, :], want_g[:, None, :], 1e-10 if dtype == np.float64 else 1e-4)
    if B <= 64:
        host_g = pysiglib_b200.sig_to_log_sig_backprop(s, w, d, N, method=0)
        assert_grad_close(host_g[:, None, :], want_g[:, None, :], 1e-10 if dtype == np.float64 else 1e-4)


@pytest.mark.parametrize("B,d,N", CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_lyndon_word_log_and_backprop(B, d, N, dtype, scalar_term):
    import pysiglib_b200
    s = _sigs(B + 2 * d + N, B, d, N, dtype, scalar_term)
    want = oracle.sig_to_log_sig(s, d, N, method=1)
    st = torch.tensor(s, device="cuda")
    pysiglib_b200.prepare_log_sig(d, N, 1)
    got = pysiglib_b200.sig_to_log_sig(st, d, N, method=1)
    assert got.shape == (B, pysiglib_b200.log_sig_length(d, N)) == want.shape
    # same coordinates as the expanded logarithm at the Lyndon words
    full = pysiglib_b200.sig_to_log_sig(st, d, N, method=0)
    idx = torch.tensor(oracle.lyndon_indices(d, N).astype(np.int64) - (0 if scalar_term else 1), device="cuda")
    assert torch.equal(got, full[:, idx])
    want_full = oracle.sig_to_log_sig(s, d, N, method=0)
    off = 1 if scalar_term else 0
    _assert_log_close(full.cpu().numpy()[:, off:], want_full[:, off:], s[:, off:], d, N, 1e-10 if dtype == np.float64 else 1e-5)
    np.testing.assert_array_equal(want, np.concatenate([np.zeros((B, 1), dtype=dtype), want_full[:, off:]], axis=1)
                                  [:, oracle.lyndon_indices(d, N).astype(np.int64)])

    w = np.random.default_rng(2).standard_normal(want.shape).astype(dtype)
    want_g = oracle.sig_to_log_sig_backprop(s.astype(np.float64), w.astype(np.float64), d, N, method=1)
    got_g = pysiglib_b200.sig_to_log_sig_backprop(st, torch.tensor(w, device="cuda"), d, N, method=1)
    assert_grad_close(got_g.cpu().numpy()[:, None, :], want_g[:, None, :], 1e-10 if dtype == np.float64 else 1e-4)


BASIS_CASES = [(5, 1, 4), (6, 2, 7), (4, 3, 4), (3, 4, 3), (300, 2, 5)]


@pytest.mark.parametrize("B,d,N", BASIS_CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("scalar_term", [False, True])
def test_lyndon_basis_log_and_backprop(B, d, N, dtype, scalar_term):
    import pysiglib_b200
    s = _sigs(B + 3 * d + N, B, d, N, dtype, scalar_term)
    want = oracle.sig_to_log_sig(s.astype(np.float64), d, N, method=2)
    st = torch.tensor(s, device="cuda")
    pysiglib_b200.prepare_log_sig(d, N, 2)
    got = pysiglib_b200.sig_to_log_sig(st, d, N, method=2)
    assert got.shape == want.shape == (B, pysiglib_b200.log_sig_length(d, N))
    # the Lyndon-basis coordinates rebuild the whole expanded logarithm: sum_j b_j [w_j]
    words, exps = oracle.lyndon_bracket_expansions(d, N)
    full = pysiglib_b200.sig_to_log_sig(st, d, N, method=0).cpu().numpy().astype(np.float64)
    off = 1 if scalar_term else 0
    rebuilt = np.zeros((B, oracle.sig_length(d, N, True)))
    g = got.cpu().numpy().astype(np.float64)
    for j, e in enumerate(exps):
        for w, c in e.items():
            idx = 0
            for letter in w:
                idx = idx * d + letter + 1
            rebuilt[:, idx] += c * g[:, j]
    _assert_log_close(rebuilt[:, 1:], full[:, off:], s[:, off:], d, N, 1e-9 if dtype == np.float64 else 2e-5)
    scale = np.maximum(np.abs(want).max(axis=1, keepdims=True), np.abs(s[:, off:off + d]).max(axis=1, keepdims=True) ** N / N)
    assert np.all(np.abs(g - want) <= (1e-9 if dtype == np.float64 else 3e-5) * np.maximum(scale, np.abs(want)))
    np.testing.assert_array_equal(pysiglib_b200.sig_to_log_sig(s, d, N, method=2), got.cpu().numpy())

    w = np.random.default_rng(4).standard_normal(want.shape).astype(dtype)
    want_g = oracle.sig_to_log_sig_backprop(s.astype(np.float64), w.astype(np.float64), d, N, method=2)
    got_g = pysiglib_b200.sig_to_log_sig_backprop(st, torch.tensor(w, device="cuda"), d, N, method=2)
    assert_grad_close(got_g.cpu().numpy()[:, None, :], want_g[:, None, :], 1e-9 if dtype == np.float64 else 2e-4)


@pytest.mark.parametrize("method", [0, 1, 2])
@pytest.mark.parametrize("flags", [(False, False), (True, False), (True, True)])
def test_log_sig_from_path_and_autograd(method, flags):
    from pysiglib_b200 import torch_api
    import pysiglib_b200
    ta, ll = flags
    rng = np.random.default_rng(3)
    path_np = (rng.standard_normal((4, 12, 2)).cumsum(1) * 0.3)
    path = torch.tensor(path_np, device="cuda", requires_grad=True)
    out = torch_api.log_sig(path, 3, time_aug=ta, lead_lag=ll, method=method)
    D = (4 if ll else 2) + (1 if ta else 0)
    want = oracle.sig_to_log_sig(oracle.sig(path_np, 3, time_aug=ta, lead_lag=ll), D, 3, method=method)
    np.testing.assert_allclose(out.detach().cpu().numpy(), want, rtol=1e-9, atol=1e-12)
    np.testing.assert_allclose(pysiglib_b200.log_sig(path_np, 3, time_aug=ta, lead_lag=ll, method=method), want,
                               rtol=1e-9, atol=1e-12)
    w = torch.tensor(rng.standard_normal(want.shape), device="cuda")
    (out * w).sum().backward()
    s = oracle.sig(path_np, 3, time_aug=ta, lead_lag=ll)
    ds = oracle.sig_to_log_sig_backprop(s, w.cpu().numpy(), D, 3, method=method)
    want_g = oracle.sig_backprop(path_np, s, ds, 3, time_aug=ta, lead_lag=ll)
    assert_grad_close(path.grad.cpu().numpy(), want_g, 1e-9)


def test_ito_correction_example_runs_through_log_sig():
    # the use the reference documents for method 0 with a correction (pysiglib/log_sig.py:395-425)
    import pysiglib_b200
    d, N, n_steps = 2, 3, 50
    dt = 1.0 / n_steps
    rng = np.random.default_rng(42)
    path = np.zeros((n_steps + 1, d))
    path[1:] = np.cumsum(rng.normal(0, np.sqrt(dt), (n_steps, d)), axis=0)
    corr = np.ascontiguousarray(np.broadcast_to((-0.5 * np.eye(d) * dt).reshape(1, -1), (n_steps, d * d)))
    got = pysiglib_b200.log_sig(torch.tensor(path, device="cuda"), N, correction=torch.tensor(corr, device="cuda"),
                                method=0)
    want = oracle.sig_to_log_sig(oracle.sig(path, N, correction=corr), d, N, method=0)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-9, atol=1e-12)


def test_unbuilt_methods_and_errors():
    import ctypes
    import pysiglib_b200
    from pysiglib_b200 import load_cusig
    s = torch.zeros((2, 14), dtype=torch.float64, device="cuda")
    with pytest.raises(NotImplementedError):
        pysiglib_b200.log_sig(torch.zeros((2, 4, 2), dtype=torch.float64, device="cuda"), 3, method=3)
    with pytest.raises(ValueError, match="method=3"):
        pysiglib_b200.sig_to_log_sig(s, 2, 3, method=3)
    lib = load_cusig.library()
    p = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_double))
    out = torch.zeros_like(s)
    assert lib.sig_to_log_sig_cuda_d(p(s), p(out), 2, 2, 3, 3, False) == 2
    assert "not part of this build" in load_cusig.last_error_message()
    assert lib.sig_to_log_sig_cuda_d(p(s), p(out), 2, 2, 0, 0, False) == 2
    assert "degree 0" in load_cusig.last_error_message()
    assert lib.prepare_log_sig_cuda(2, 3, 1, False) == 0
    assert lib.prepare_log_sig_cuda(2, 3, 2, False) == 0
    assert lib.prepare_log_sig_cuda(2, 3, 3, False) == 2


FUSED_CASES = [  # (B, L, d, N, flags): shapes whose biggest forward tile carries the fused log-signature sweep
    (5, 40, 16, 4, {}),                       # 16 warps per path: a cluster of 4 CTAs shares the lower levels
    (9, 33, 8, 4, {}),                        # float32: one warp per path, four paths per CTA
    (6, 30, 3, 4, {"time_aug": True}),
    (3, 20, 4, 3, {"lead_lag": True}),
    (300, 20, 16, 4, {}),
    (70000, 5, 3, 3, {}),                     # more CTAs than one grid row of paths
]


@pytest.mark.parametrize("case", FUSED_CASES, ids=lambda c: "B%d_L%d_d%d_N%d%s" % (c[:4] + ("".join("_" + k for k in c[4]),)))
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("method", [0, 1, 2])
def test_fused_log_sweep_matches_the_two_step_route_and_the_oracle(case, dtype, method):
    """log_sig in one launch: the forward sweep publishes the levels below N in (distributed) shared
    memory and turns its level-N registers into the logarithm; the signature never reaches global
    memory.  Forced through the test hook (the automatic rule only picks it for short paths), checked
    against the route through scratch and against the oracle."""
    import pysiglib_b200
    from pysiglib_b200 import load_cusig
    B, L, d, N, kw = case
    D = (2 * d if kw.get("lead_lag") else d) + (1 if kw.get("time_aug") else 0)
    path = brownian_paths(B % 97 + L + d, B, L, d, dtype) * 1.2
    x = torch.tensor(path, device="cuda")
    scalar = method == 0 and B == 9
    pysiglib_b200.prepare_log_sig(D, N, method)
    load_cusig.set_kernel_policy(1)   # generic kernels: the signature goes to scratch, then the tensor-log kernels
    try:
        two_step = pysiglib_b200.log_sig(x, N, method=method, scalar_term=scalar, **kw)
    finally:
        load_cusig.set_kernel_policy(0)
    load_cusig.set_tile_preference(1)
    try:
        before = load_cusig.launch_count()
        fused = pysiglib_b200.log_sig(x, N, method=method, scalar_term=scalar, **kw)
        launches = load_cusig.launch_count() - before
    finally:
        load_cusig.set_tile_preference(0)
    assert launches == (2 if method == 2 else 1), "the fused sweep did not run (%d launches)" % launches
    assert fused.shape == two_step.shape
    n = min(B, 8)
    sig64 = oracle.sig(path[:n].astype(np.float64), N, **kw)
    want = oracle.sig_to_log_sig(sig64, D, N, method=method)
    got, ref = fused[:n].cpu().numpy(), two_step[:n].cpu().numpy()
    if scalar:
        assert np.all(got[:, 0] == 0)
        got, ref = got[:, 1:], ref[:, 1:]
    tol = 1e-10 if dtype == np.float64 else 2e-5
    if method == 0:
        _assert_log_close(got, want, sig64, D, N, tol)
        _assert_log_close(ref, want, sig64, D, N, tol)
    else:
        scale = np.maximum(np.abs(sig64).max(axis=1, keepdims=True), 1.0) * (1.0 if method == 1 else 10.0)
        assert np.all(np.abs(got - want) <= tol * scale), np.abs(got - want).max()
        assert np.all(np.abs(ref - want) <= tol * scale)
    # the whole batch agrees with the two-step route to rounding
    scale_all = float(two_step.abs().max()) + 1e-30
    assert float((fused - two_step).abs().max()) <= (1e-11 if dtype == np.float64 else 3e-5) * max(scale_all, 1.0)


# Batches of at least one signature per SM take the one-CTA-per-signature kernels of sig_log_stream.cu:
# the forward for any dimension, the backward for power-of-two dimensions (partial levels, several
# iterations per level, register sums that are flushed mid-level, every vector width - the scalar term
# shifts the alignment - and every method).
STREAMED_CASES = [(150, 2, 2), (150, 2, 6), (200, 2, 8), (150, 4, 3), (150, 4, 5), (150, 4, 6), (150, 8, 3), (150, 8, 4),
                  (150, 16, 2), (150, 16, 3), (148, 16, 4), (150, 32, 2), (150, 3, 4), (150, 5, 3), (160, 6, 3), (150, 1, 4)]


@pytest.mark.parametrize("B,d,N", STREAMED_CASES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("scalar_term", [False, True])
@pytest.mark.parametrize("method", [0, 1, 2])
def test_streamed_log_and_backprop(B, d, N, dtype, scalar_term, method):
    import pysiglib_b200
    from pysiglib_b200 import load_cusig
    if method == 2 and d ** N > 70000:
        pytest.skip("the basis change of this shape is slow to prepare on the host")
    s = _sigs(B + d + N, B, d, N, dtype, scalar_term)
    st = torch.tensor(s, device="cuda")
    pysiglib_b200.prepare_log_sig(d, N, method)
    off = 1 if scalar_term else 0

    before = load_cusig.launch_count()
    got = pysiglib_b200.sig_to_log_sig(st, d, N, method=method)
    launches = load_cusig.launch_count() - before
    assert launches == (2 if method == 2 else 1), "expected the one-kernel forward, saw %d launches" % launches
    want = oracle.sig_to_log_sig(s.astype(np.float64) if method == 2 else s, d, N, method=method)
    rtol = 1e-10 if dtype == np.float64 else 1e-5
    if method == 0:
        _assert_log_close(got.cpu().numpy()[:, off:], want[:, off:], s[:, off:], d, N, rtol)
        if scalar_term:
            assert torch.all(got[:, 0] == 0)
    else:
        scale = np.maximum(np.abs(want).max(axis=1, keepdims=True),
                           np.abs(s[:, off:off + d]).max(axis=1, keepdims=True).astype(np.float64) ** N / N)
        assert (np.abs(got.cpu().numpy() - want) / scale).max() <= (1e-9 if dtype == np.float64 else 3e-5)

    M = s.shape[1] if method == 0 else pysiglib_b200.log_sig_length(d, N)
    w = np.random.default_rng(2).standard_normal((B, M)).astype(dtype)
    want_g = oracle.sig_to_log_sig_backprop(s.astype(np.float64), w.astype(np.float64), d, N, method=method)
    before = load_cusig.launch_count()
    got_g = pysiglib_b200.sig_to_log_sig_backprop(st, torch.tensor(w, device="cuda"), d, N, method=method)
    launches = load_cusig.launch_count() - before
    if d & (d - 1) == 0 and d >= 2:
        assert launches <= 2, "expected the one-kernel backward (plus the basis pull-back for method 2), saw %d launches" % launches
    assert_grad_close(got_g.cpu().numpy()[:, None, :], want_g[:, None, :], 1e-10 if dtype == np.float64 else 1e-4)
    if scalar_term:
        assert not got_g[:, 0].any()
