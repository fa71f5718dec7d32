"""Same-GPU parity against the reference's own CUDA kernels (oracle/_ref/libcusig_ref.so,
built from the reference's unmodified sources by oracle/build_ref_cuda.sh).  Skipped when
that library has not been built."""
import numpy as np
import pytest
import torch

from oracle import refcuda
from conftest import assert_grad_parity, assert_sig_close, brownian_paths
from oracle import oracle

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not refcuda.available(), reason="reference CUDA library not built")]

# the five benchmark shapes at reduced batch / length, plus flag cases
CASES = [  # (B, L, d, N, time_aug, lead_lag, dtype)
    (4, 200, 10, 5, False, False, np.float64),
    (16, 256, 2, 12, False, False, np.float64),
    (4, 300, 5, 7, False, False, np.float32),
    (8, 400, 8, 4, False, False, np.float32),
    (8, 300, 16, 4, False, False, np.float32),
    (3, 50, 3, 4, True, True, np.float64),
    (3, 60, 8, 3, True, False, np.float32),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "B%d_L%d_d%d_N%d_%d%d_%s" % (c[:6] + (c[6].__name__,)))
def test_forward_and_backward_match_reference_cuda(case):
    import pysiglib_b200
    B, L, d, N, ta, ll, dtype = case
    path_np = brownian_paths(B + L + d, B, L, d, dtype)
    path = torch.tensor(path_np, device="cuda")
    kw = dict(time_aug=ta, lead_lag=ll, end_time=1.3)
    D = (2 * d if ll else d) + (1 if ta else 0)
    ref = refcuda.sig(path, N, **kw)
    ours = pysiglib_b200.sig(path, N, **kw)
    rtol = 1e-10 if dtype == np.float64 else 1e-5
    assert_sig_close(ours.cpu().numpy(), ref.cpu().numpy(), D, N, rtol)

    seeds = torch.randn(ref.shape, dtype=ref.dtype, device="cuda", generator=torch.Generator("cuda").manual_seed(B))
    ref_g = refcuda.sig_backprop(path, ref, seeds, N, **kw)
    our_g = pysiglib_b200.sig_backprop(path, ref, seeds, N, **kw)
    p64 = path_np.astype(np.float64)
    truth = oracle.sig_backprop(p64, oracle.sig(p64, N, **kw), seeds.cpu().numpy().astype(np.float64), N, **kw)
    assert_grad_parity(our_g.cpu().numpy(), ref_g.cpu().numpy(), truth, rtol)


@pytest.mark.parametrize("time_aug,lead_lag", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_transform_path_matches_reference_cuda(time_aug, lead_lag, dtype):
    """The standalone path transform and its backward against the reference's own kernels
    (siglib/cusig/cu_path_transforms.cu:100-205): pure data movement, so bit-identical."""
    import pysiglib_b200
    B, L, d = 5, 23, 3
    path = torch.tensor(brownian_paths(4, B, L, d, dtype), device="cuda")
    kw = dict(time_aug=time_aug, lead_lag=lead_lag, end_time=0.7)
    ref = refcuda.transform_path(path, **kw)
    ours = pysiglib_b200.transform_path(path, **kw)
    assert ours.shape == ref.shape
    tol = 0 if not time_aug else (1e-15 if dtype == np.float64 else 1e-6)  # the time channel is k * dt either way
    assert float((ours - ref).abs().max()) <= tol
    derivs = torch.randn(ref.shape, dtype=ref.dtype, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    ref_g = refcuda.transform_path_backprop(derivs, L, d, **kw)
    our_g = pysiglib_b200.transform_path_backprop(derivs, **kw)
    assert our_g.shape == ref_g.shape == path.shape
    scale = float(ref_g.abs().max())
    assert float((our_g - ref_g).abs().max()) <= (1e-14 if dtype == np.float64 else 1e-6) * scale
