"""The allocation-free backward entry point (sigb200_sig_backprop_noalloc_*).

It serves hosts that cannot allocate device memory when the gradient is needed (their own
allocator owns the GPU's memory, or they cannot afford the device-wide synchronisation of
cudaMalloc / cudaFree).  Its scratch is a static buffer inside the library that every call
shares, so the test calls it twice in a row with different data: the second result must not
be polluted by what the first call left behind.  Each result is compared with the regular
entry point (sig_backprop_cuda_*) through the C ABI.

Collected last on purpose (file name), so that a run stopping at the first failure has
already executed every other test."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import brownian_paths
from pysiglib_b200 import load_cusig

pytestmark = pytest.mark.gpu


def _ptr(t, real):
    return ctypes.cast(t.data_ptr(), ctypes.POINTER(real))


def _backprop(symbol, path, sig, derivs, degree, extra):
    name = str(path.dtype).replace("torch.", "")
    real = ctypes.c_float if name == "float32" else ctypes.c_double
    B, L, d = path.shape
    out = torch.full_like(path, -7.0)
    fn = load_cusig.fn(symbol, name)
    args = [_ptr(path, real), _ptr(out, real), _ptr(derivs, real), _ptr(sig, real), B, d, L, degree, False, False,
            real(1.0), False] + extra
    code = fn(*args)
    assert code == 0, load_cusig.last_error_message()
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("dtype,tol", [(np.float32, 1e-5), (np.float64, 1e-10)])
def test_noalloc_backprop_matches_regular_entry_point_twice(dtype, tol):
    lib = load_cusig.library()
    assert lib.sigb200_noalloc_scratch_bytes() == 32 << 20
    import pysiglib_b200
    for call, (seed, B, L) in enumerate([(21, 6, 70), (22, 3, 33)]):
        path = torch.tensor(brownian_paths(seed, B, L, 8, dtype), device="cuda")
        sig = pysiglib_b200.sig(path, 4)
        derivs = torch.randn(sig.shape, dtype=sig.dtype, device="cuda", generator=torch.Generator("cuda").manual_seed(seed))
        want = _backprop("sig_backprop_cuda", path, sig, derivs, 4, [None, 0, 0, 0])
        got = _backprop("sigb200_sig_backprop_noalloc", path, sig, derivs, 4, [ctypes.c_void_p(None), 1])
        scale = want.abs().amax(dim=(1, 2), keepdim=True)
        err = ((got - want).abs() / scale).max().item()
        assert err <= tol, "call %d: %.3e" % (call, err)


def test_noalloc_rejects_what_it_cannot_serve():
    lib = load_cusig.library()
    path = torch.zeros((1, 4, 8), device="cuda")
    sig = torch.zeros((1, 4680), device="cuda")
    out = torch.zeros_like(path)
    f32 = ctypes.c_float
    # more scratch than the static buffer holds: batch * (L - 1) * d * 4 bytes > 32 MiB
    code = lib.sigb200_sig_backprop_noalloc_f(_ptr(path, f32), _ptr(out, f32), _ptr(sig, f32), _ptr(sig, f32),
                                              1 << 20, 8, 4, 4, False, False, 1.0, False, None, 1)
    assert code == 2 and "static" in load_cusig.last_error_message()
    # a shape outside the register-tile table
    code = lib.sigb200_sig_backprop_noalloc_f(_ptr(path, f32), _ptr(out, f32), _ptr(sig, f32), _ptr(sig, f32),
                                              1, 8, 4, 9, False, False, 1.0, False, None, 1)
    assert code == 2 and "register-tile" in load_cusig.last_error_message()
    # host pointers
    host = np.zeros((1, 4, 8), dtype=np.float32)
    hp = host.ctypes.data_as(ctypes.POINTER(f32))
    code = lib.sigb200_sig_backprop_noalloc_f(hp, hp, hp, hp, 1, 8, 4, 4, False, False, 1.0, False, None, 1)
    assert code == 2 and "device pointers" in load_cusig.last_error_message()
