"""The timed CPU baseline (oracle/timing.py: -O3 -march=native build, SIMD-across-paths forward)
computes the same numbers as the checker up to rounding; it is only ever timed, never used as
a checker, but a baseline that computed something else would not be a baseline."""
import numpy as np
import pytest

from conftest import assert_sig_close, brownian_paths
from oracle import oracle, timing


@pytest.mark.parametrize("dtype,B,L,d,N,batch_simd", [(np.float64, 9, 40, 2, 6, True), (np.float32, 19, 33, 3, 4, True),
                                                      (np.float64, 3, 20, 2, 5, False), (np.float32, 5, 30, 8, 3, False),
                                                      (np.float64, 6, 17, 3, 4, True), (np.float64, 6, 17, 4, 3, False)])
def test_timing_build_matches_the_checker(dtype, B, L, d, N, batch_simd):
    path = brownian_paths(B + L, B, L, d, dtype)
    assert timing.takes_batch_simd(B, L, d, N, dtype) == batch_simd
    got, variant = timing.sig(path, N, n_threads=3)
    assert variant == ("SIMD across paths" if batch_simd else "per-path Horner")
    want = oracle.sig(path, N)
    assert_sig_close(got, want, d, N, 1e-12 if dtype == np.float64 else 2e-5)
    seeds = np.random.default_rng(1).standard_normal(want.shape).astype(dtype)
    g = timing.sig_backprop(path, want, seeds, N, n_threads=2)
    g_want = oracle.sig_backprop(path, want, seeds, N)
    scale = np.abs(g_want).max()
    assert np.abs(g - g_want).max() <= (1e-11 if dtype == np.float64 else 3e-4) * scale
