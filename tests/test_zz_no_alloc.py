"""The allocation-free backward entry point (sigb200_sig_backprop_noalloc_*).

It serves hosts that cannot allocate device memory when the gradient is needed (their own
allocator owns the GPU's memory, or they cannot afford the device-wide synchronisation of
cudaMalloc / cudaFree).  Its scratch is a static buffer inside the library that every call
shares, so the test calls it twice in a row with different data: the second result must not
be polluted by what the first call left behind.  Each result is compared with the regular
entry point (sig_backprop_cuda_*) through the C ABI and with the CPU oracle, and a repeated
call of a shape is checked to leave the device's free memory and the stream-ordered pool's
reservation untouched.

Collected last on purpose (file name), so that a run stopping at the first failure has
already executed every other test."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import assert_grad_parity, brownian_paths
from oracle import oracle
from pysiglib_b200 import load_cusig

pytestmark = pytest.mark.gpu


def _ptr(t, real):
    return ctypes.cast(t.data_ptr(), ctypes.POINTER(real))


def _backprop(symbol, path, sig, derivs, degree, extra, time_aug=False, lead_lag=False, out=None):
    name = str(path.dtype).replace("torch.", "")
    real = ctypes.c_float if name == "float32" else ctypes.c_double
    B, L, d = path.shape
    out = torch.full_like(path, -7.0) if out is None else out
    fn = load_cusig.fn(symbol, name)
    args = [_ptr(path, real), _ptr(out, real), _ptr(derivs, real), _ptr(sig, real), B, d, L, degree, time_aug, lead_lag,
            real(1.0), False] + extra
    code = fn(*args)
    assert code == 0, load_cusig.last_error_message()
    torch.cuda.synchronize()
    return out


def _pool_reserved():
    """Bytes the device's default stream-ordered pool (the one cudaMallocAsync draws from) holds."""
    dev = torch.cuda.current_device()
    try:
        from cuda.bindings import runtime as rt
    except ImportError:
        try:
            from cuda import cudart as rt
        except ImportError:
            return None
    err, pool = rt.cudaDeviceGetDefaultMemPool(dev)
    if int(err) != 0:
        return None
    err, value = rt.cudaMemPoolGetAttribute(pool, rt.cudaMemPoolAttr.cudaMemPoolAttrReservedMemCurrent)
    return int(value) if int(err) == 0 else None


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
        # and against the CPU oracle, not only against the same kernel through the other door
        p64 = path.cpu().numpy().astype(np.float64)
        s64 = oracle.sig(p64, 4)
        d64 = derivs.cpu().numpy().astype(np.float64)
        truth = oracle.sig_backprop(p64, s64, d64, 4)
        same = oracle.sig_backprop(path.cpu().numpy(), sig.cpu().numpy(), derivs.cpu().numpy(), 4)
        assert_grad_parity(got.cpu().numpy(), same, truth, tol, "no-alloc call %d" % call)


@pytest.mark.parametrize("dtype,tol", [(np.float32, 1e-5), (np.float64, 1e-10)])
def test_noalloc_with_flags_on_a_side_stream_allocates_nothing(dtype, tol):
    """time_aug + lead_lag (the kernels that synthesise increments), a non-default stream and
    synchronize = 0; the second call of the shape must leave the free device memory and the
    stream-ordered pool's reservation exactly as it found them."""
    import pysiglib_b200
    B, L, d, N = 5, 41, 2, 3
    path = torch.tensor(brownian_paths(31, B, L, d, dtype), device="cuda")
    sig = pysiglib_b200.sig(path, N, time_aug=True, lead_lag=True)
    derivs = torch.randn(sig.shape, dtype=sig.dtype, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    want = _backprop("sig_backprop_cuda", path, sig, derivs, N, [None, 0, 0, 0], True, True)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    extra = [ctypes.c_void_p(side.cuda_stream), 0]
    out = torch.full_like(path, -7.0)
    _backprop("sigb200_sig_backprop_noalloc", path, sig, derivs, N, extra, True, True, out)  # warm-up: loads code
    torch.cuda.synchronize()
    free_before, reserved_before = torch.cuda.mem_get_info()[0], _pool_reserved()
    out.fill_(-7.0)
    torch.cuda.synchronize()
    got = _backprop("sigb200_sig_backprop_noalloc", path, sig, derivs, N, extra, True, True, out)
    side.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert _pool_reserved() == reserved_before
    scale = want.abs().amax(dim=(1, 2), keepdim=True)
    assert ((got - want).abs() / scale).max().item() <= tol
    p64 = path.cpu().numpy().astype(np.float64)
    s64 = oracle.sig(p64, N, time_aug=True, lead_lag=True)
    truth = oracle.sig_backprop(p64, s64, derivs.cpu().numpy().astype(np.float64), N, time_aug=True, lead_lag=True)
    same = oracle.sig_backprop(path.cpu().numpy(), sig.cpu().numpy(), derivs.cpu().numpy(), N, time_aug=True,
                               lead_lag=True)
    assert_grad_parity(got.cpu().numpy(), same, truth, tol, "no-alloc with flags")


def test_noalloc_degree_one_needs_no_tile():
    import pysiglib_b200
    path = torch.tensor(brownian_paths(5, 3, 9, 40, np.float64), device="cuda")
    sig = pysiglib_b200.sig(path, 1)
    derivs = torch.randn(sig.shape, dtype=sig.dtype, device="cuda", generator=torch.Generator("cuda").manual_seed(4))
    want = _backprop("sig_backprop_cuda", path, sig, derivs, 1, [None, 0, 0, 0])
    got = _backprop("sigb200_sig_backprop_noalloc", path, sig, derivs, 1, [ctypes.c_void_p(None), 1])
    assert torch.equal(got, want)


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
    # a host signature or host seeds next to device path / out: rejected on the host, nothing is launched
    host_sig = np.zeros((1, 4680), dtype=np.float32)
    hs = host_sig.ctypes.data_as(ctypes.POINTER(f32))
    before = load_cusig.launch_count()
    code = lib.sigb200_sig_backprop_noalloc_f(_ptr(path, f32), _ptr(out, f32), _ptr(sig, f32), hs,
                                              1, 8, 4, 4, False, False, 1.0, False, None, 1)
    assert code == 2 and "device pointers" in load_cusig.last_error_message()
    code = lib.sigb200_sig_backprop_noalloc_f(_ptr(path, f32), _ptr(out, f32), hs, _ptr(sig, f32),
                                              1, 8, 4, 4, False, False, 1.0, False, None, 1)
    assert code == 2 and "device pointers" in load_cusig.last_error_message()
    assert load_cusig.launch_count() == before
    torch.cuda.synchronize()
