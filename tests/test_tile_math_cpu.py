"""CPU check of the register-tile arithmetic used by the CUDA kernels.

``tests/cpu_harness/tile_harness.cpp`` compiles ``pysiglib_b200/csrc/tile_math.h``
for the host and runs every execution unit of a path sequentially.  Forward and
backward results must agree with the oracle; this validates the unit decomposition,
the indexing and the partial-adjoint scheme without a GPU."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "cpu_harness", "tile_harness.cpp")
HDR = os.path.join(HERE, "..", "pysiglib_b200", "csrc", "tile_math.h")
LIB = os.path.join(HERE, "cpu_harness", "_build", "tile_harness.so")

SHAPES = [(2, 2, 1, 2), (2, 2, 0, 2), (2, 5, 2, 2), (2, 5, 3, 1), (2, 6, 1, 1), (3, 3, 0, 3), (3, 3, 2, 1),
          (3, 4, 1, 3), (3, 4, 2, 3), (4, 3, 1, 2), (4, 4, 2, 4), (5, 3, 1, 5), (6, 3, 1, 3), (8, 3, 1, 4),
          (3, 7, 5, 3), (4, 6, 4, 2), (2, 8, 6, 1)]


@pytest.fixture(scope="module")
def harness():
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < max(os.path.getmtime(SRC), os.path.getmtime(HDR)):
        subprocess.run(["g++", "-O1", "-std=c++17", "-ffp-contract=off", "-mfma", "-fPIC", "-shared",
                        "-o", LIB, SRC], check=True)
    return ctypes.CDLL(LIB)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_tile_forward_and_backward(harness, shape, dtype):
    D, N, P, G = shape
    suf = "d" if dtype == np.float64 else "f"
    real = ctypes.c_double if dtype == np.float64 else ctypes.c_float
    ptr = ctypes.POINTER(real)
    rng = np.random.default_rng(D * 1000 + N * 100 + P * 10 + G)
    L = 7
    path = np.ascontiguousarray(rng.normal(scale=0.5, size=(L, D)).astype(dtype))
    n = oracle.sig_length(D, N)
    out = np.zeros(n, dtype=dtype)
    getattr(harness, "fwd_%s_%d_%d_%d_%d" % (suf, D, N, P, G))(
        path.ctypes.data_as(ptr), L, out.ctypes.data_as(ptr))
    expect = oracle.sig(path, N)
    if dtype == np.float64:
        np.testing.assert_allclose(out, expect, rtol=1e-13, atol=1e-15)
    else:
        # same operation order as the reference's CPU code: float32 results are bit-identical
        np.testing.assert_array_equal(out, expect)

    seeds = np.ascontiguousarray(rng.normal(size=n).astype(dtype))
    grad = np.zeros_like(path)
    getattr(harness, "bwd_%s_%d_%d_%d_%d" % (suf, D, N, P, G))(
        path.ctypes.data_as(ptr), L, expect.ctypes.data_as(ptr), seeds.ctypes.data_as(ptr),
        grad.ctypes.data_as(ptr))
    want = oracle.sig_backprop(path, expect, seeds, N)
    tol = 1e-11 if dtype == np.float64 else 2e-4
    np.testing.assert_allclose(grad, want, rtol=tol, atol=tol * np.abs(want).max())


@pytest.mark.parametrize("shape", SHAPES)
def test_tile_log_epilogue(harness, shape):
    """The log-signature epilogue of the fused forward sweep (log_prefix_weights / tile_log_top /
    log_low_prefix) against the oracle's tensor logarithm of the same signature."""
    D, N, P, G = shape
    rng = np.random.default_rng(D * 77 + N * 5 + P)
    L = 6
    path = np.ascontiguousarray(rng.normal(scale=0.6, size=(L, D)))
    n = oracle.sig_length(D, N)
    out = np.zeros(n)
    getattr(harness, "log_d_%d_%d_%d_%d" % (D, N, P, G))(path.ctypes.data_as(ctypes.POINTER(ctypes.c_double)), L,
                                                       out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)))
    want = oracle.sig_to_log_sig(oracle.sig(path, N), D, N, method=0)
    scale = np.abs(oracle.sig(path, N)).max()
    np.testing.assert_allclose(out, want, rtol=1e-10, atol=1e-12 * max(scale, 1.0))
