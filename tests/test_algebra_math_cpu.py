"""CPU check of the per-coefficient tensor-algebra arithmetic used by the CUDA kernels.

``tests/cpu_harness/algebra_harness.cpp`` compiles ``pysiglib_b200/csrc/algebra_math.h`` for
the host and runs the phases of the CUDA kernels as plain loops; results must agree with the
oracle.  This validates the indexing of products, adjoints, the exponential and its adjoint,
and the way the corrected-signature kernels chain them, without a GPU."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "cpu_harness", "algebra_harness.cpp")
HDR = os.path.join(HERE, "..", "pysiglib_b200", "csrc", "algebra_math.h")
LIB = os.path.join(HERE, "cpu_harness", "_build", "algebra_harness.so")

SHAPES = [(1, 4), (2, 2), (2, 5), (3, 3), (3, 4), (5, 3), (4, 1)]
U64 = ctypes.c_uint64


@pytest.fixture(scope="module")
def harness():
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < max(os.path.getmtime(SRC), os.path.getmtime(HDR)):
        subprocess.run(["g++", "-O1", "-std=c++17", "-ffp-contract=off", "-mfma", "-fPIC", "-shared",
                        "-o", LIB, SRC], check=True)
    return ctypes.CDLL(LIB)


def _call(harness, name, dtype, *args):
    suf, real = ("d", ctypes.c_double) if dtype == np.float64 else ("f", ctypes.c_float)
    conv = [a.ctypes.data_as(ctypes.POINTER(real)) if isinstance(a, np.ndarray) else U64(a) for a in args]
    getattr(harness, "%s_%s" % (name, suf))(*conv)


def _tol(dtype):
    return dict(rtol=1e-12, atol=1e-13) if dtype == np.float64 else dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dim,degree", SHAPES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_exp_and_its_adjoint(harness, dim, degree, dtype):
    rng = np.random.default_rng(dim * 10 + degree)
    n = oracle.sig_length(dim, degree)
    x = (rng.standard_normal(n) * 0.5).astype(dtype)
    e = np.zeros(n, dtype=dtype)
    _call(harness, "alg_exp", dtype, x, e, dim, degree)
    full = np.concatenate([[0], x]).astype(dtype)
    np.testing.assert_allclose(e, oracle.tensor_exp(full, dim, degree)[1:], **_tol(dtype))

    w = rng.standard_normal(n).astype(dtype)
    g = np.zeros(dim, dtype=dtype)
    _call(harness, "alg_exp_adjoint_level1", dtype, x, w, g, dim, degree)
    want = oracle.tensor_exp_backprop(np.concatenate([[0], w]).astype(dtype), full, dim, degree)[1:1 + dim]
    np.testing.assert_allclose(g, want, **_tol(dtype))


@pytest.mark.parametrize("dim,degree", SHAPES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_product_and_adjoints(harness, dim, degree, dtype):
    rng = np.random.default_rng(100 + dim * 10 + degree)
    n = oracle.sig_length(dim, degree)
    a, b, g = [(rng.standard_normal(n) * 0.5).astype(dtype) for _ in range(3)]
    c = np.zeros(n, dtype=dtype)
    _call(harness, "alg_product", dtype, a, b, c, dim, degree)
    np.testing.assert_allclose(c, oracle.sig_combine(a, b, dim, degree), **_tol(dtype))
    da, db = np.zeros(n, dtype=dtype), np.zeros(n, dtype=dtype)
    _call(harness, "alg_adjoints", dtype, g, a, b, da, db, dim, degree)
    wa, wb = oracle.sig_combine_backprop(g, a, b, dim, degree)
    np.testing.assert_allclose(da, wa, **_tol(dtype))
    np.testing.assert_allclose(db, wb, **_tol(dtype))


@pytest.mark.parametrize("dim,degree", SHAPES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_linear_sig_and_adjoint(harness, dim, degree, dtype):
    rng = np.random.default_rng(200 + dim * 10 + degree)
    n = oracle.sig_length(dim, degree)
    v = rng.standard_normal(dim).astype(dtype)
    out = np.zeros(n, dtype=dtype)
    _call(harness, "alg_linear_sig", dtype, v, out, dim, degree)
    expect = oracle.linear_sig(v, degree)
    if dtype == np.float32:
        np.testing.assert_array_equal(out, expect)  # same operations in the same order
    else:
        np.testing.assert_allclose(out, expect, rtol=1e-15)
    # adjoint: join onto the empty signature so that d_out passes straight to the linear part
    g = rng.standard_normal(n).astype(dtype)
    dv = np.zeros(dim, dtype=dtype)
    _call(harness, "alg_linear_sig_adjoint", dtype, v, g, dv, dim, degree)
    _, want = oracle.sig_join_backprop(g, np.zeros(n, dtype=dtype), v, dim, degree)
    np.testing.assert_allclose(dv, want, **_tol(dtype))


@pytest.mark.parametrize("dim,degree", SHAPES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_tensor_log_and_its_adjoint(harness, dim, degree, dtype):
    rng = np.random.default_rng(400 + dim * 10 + degree)
    n = oracle.sig_length(dim, degree)
    x = (rng.standard_normal(n) * 0.5).astype(dtype)
    y = np.zeros(n, dtype=dtype)
    _call(harness, "alg_log", dtype, x, y, dim, degree)
    np.testing.assert_allclose(y, oracle.sig_to_log_sig(x, dim, degree, method=0), **_tol(dtype))
    w = rng.standard_normal(n).astype(dtype)
    dx = np.zeros(n, dtype=dtype)
    _call(harness, "alg_log_backprop", dtype, x, w, dx, dim, degree)
    np.testing.assert_allclose(dx, oracle.sig_to_log_sig_backprop(x, w, dim, degree, method=0), **_tol(dtype))


@pytest.mark.parametrize("dim,degree,levels", [(1, 4, 3), (2, 3, 1), (2, 4, 3), (3, 3, 2)])
@pytest.mark.parametrize("layout", ["constant", "per_segment"])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_corrected_signature_chain(harness, dim, degree, levels, layout, dtype):
    rng = np.random.default_rng(300 + dim * 10 + degree)
    L = 6
    path = (rng.standard_normal((L, dim)).cumsum(0) * 0.4).astype(dtype)
    clen = sum(dim ** k for k in range(2, 2 + levels))
    corr = (rng.standard_normal((L - 1, clen)) * 0.2).astype(dtype)
    if layout == "constant":
        corr, stride = np.ascontiguousarray(corr[0]), 0
    else:
        stride = clen
    n = oracle.sig_length(dim, degree)
    out = np.zeros(n, dtype=dtype)
    _call(harness, "alg_correction_forward", dtype, path, L, dim, degree, corr, clen, stride, out)
    expect = oracle.sig(path, degree, correction=corr)
    np.testing.assert_allclose(out, expect, **_tol(dtype))

    w = rng.standard_normal(n).astype(dtype)
    grad = np.zeros_like(path)
    _call(harness, "alg_correction_backward", dtype, path, L, dim, degree, corr, clen, stride, expect, w, grad)
    want = oracle.sig_backprop(path, expect, w, degree, correction=corr)
    tol = dict(rtol=1e-10, atol=1e-11) if dtype == np.float64 else dict(rtol=2e-4, atol=2e-4)
    np.testing.assert_allclose(grad, want, **tol)
