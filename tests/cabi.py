"""Test helper: calls libcusig.so through its C ABI exactly as a ctypes client of the
reference would (reference-named symbols, raw pointers), for host or device buffers."""
import ctypes

import numpy as np

from pysiglib_b200 import load_cusig


def _ptr(arr, real):
    if arr is None:
        return ctypes.POINTER(real)()
    if isinstance(arr, np.ndarray):
        return arr.ctypes.data_as(ctypes.POINTER(real))
    return ctypes.cast(arr.data_ptr(), ctypes.POINTER(real))  # torch tensor


def _real(dtype_name):
    return ctypes.c_float if dtype_name == "float32" else ctypes.c_double


def _dtype_name(arr):
    return str(arr.dtype).replace("torch.", "")


def aug_dim(d, time_aug, lead_lag):
    return (2 * d if lead_lag else d) + (1 if time_aug else 0)


def sig_len(d, degree, time_aug=False, lead_lag=False, scalar_term=False):
    n = load_cusig.library().sigb200_sig_length(aug_dim(d, time_aug, lead_lag), degree)
    return n - (0 if scalar_term else 1)


def signature_cuda(path, degree, *, time_aug=False, lead_lag=False, end_time=1.0, horner=True,
                   scalar_term=False, out=None, pad=0):
    """signature_cuda_{f,d} on a (B, L, d) numpy array or torch tensor; returns (code, out).
    ``pad`` extra elements are allocated after the output and preset to -1 (sentinel)."""
    name = _dtype_name(path)
    real = _real(name)
    B, L, d = path.shape
    n = sig_len(d, degree, time_aug, lead_lag, scalar_term)
    if out is None:
        if isinstance(path, np.ndarray):
            out = np.full(B * n + pad, -1.0, dtype=path.dtype)
        else:
            import torch
            out = torch.full((B * n + pad,), -1.0, dtype=path.dtype, device=path.device)
    code = load_cusig.fn("signature_cuda", name)(
        _ptr(path, real), _ptr(out, real), B, d, L, degree, time_aug, lead_lag, real(end_time), horner,
        scalar_term, _ptr(None, real), 0, 0, 0)
    return code, out


def sig_backprop_cuda(path, sig, derivs, degree, *, time_aug=False, lead_lag=False, end_time=1.0,
                      scalar_term=False, pad=0):
    name = _dtype_name(path)
    real = _real(name)
    B, L, d = path.shape
    if isinstance(path, np.ndarray):
        out = np.full(B * L * d + pad, -1.0, dtype=path.dtype)
    else:
        import torch
        out = torch.full((B * L * d + pad,), -1.0, dtype=path.dtype, device=path.device)
    code = load_cusig.fn("sig_backprop_cuda", name)(
        _ptr(path, real), _ptr(out, real), _ptr(derivs, real), _ptr(sig, real), B, d, L, degree, time_aug,
        lead_lag, real(end_time), scalar_term, _ptr(None, real), 0, 0, 0)
    return code, out
