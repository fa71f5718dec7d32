"""Checker and timed baseline (test infrastructure, never used by the product): the reference's own CUDA kernels, built unmodified from its two
translation units by oracle/build_ref_cuda.sh into oracle/_ref/libcusig_ref.so.  Used only as
a checker and as a timed baseline; absent file -> callers skip."""
import ctypes
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "oracle", "_ref", "libcusig_ref.so")
_lib = None


def available():
    return os.path.exists(PATH)


def library():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(PATH)
        u64, b = ctypes.c_uint64, ctypes.c_bool
        for suf, real in (("f", ctypes.c_float), ("d", ctypes.c_double)):
            p = ctypes.POINTER(real)
            f = getattr(lib, "signature_cuda_" + suf)
            f.argtypes = (p, p, u64, u64, u64, u64, b, b, real, b, b, p, u64, u64, u64)
            f.restype = ctypes.c_int
            g = getattr(lib, "sig_backprop_cuda_" + suf)
            g.argtypes = (p, p, p, p, u64, u64, u64, u64, b, b, real, b, p, u64, u64, u64)
            g.restype = ctypes.c_int
            for name in ("transform_path_cuda_", "transform_path_backprop_cuda_"):
                t = getattr(lib, name + suf)
                t.argtypes = (p, p, u64, u64, u64, b, b, real)
                t.restype = ctypes.c_int
        _lib = lib
    return _lib


def _real(t):
    import torch
    return ctypes.c_float if t.dtype == torch.float32 else ctypes.c_double


def _ptr(t):
    return ctypes.cast(t.data_ptr(), ctypes.POINTER(_real(t)))


def _correction_args(correction, B, L):
    """(pointer, length, batch stride, segment stride) for a contiguous CUDA tensor of shape (C,),
    (L-1, C) or (B, L-1, C), or the empty correction."""
    if correction is None or correction.numel() == 0:
        return None, 0, 0, 0
    c = correction.shape[-1]
    if correction.dim() == 1:
        return _ptr(correction), c, 0, 0
    if correction.dim() == 2:
        return _ptr(correction), c, 0, c
    return _ptr(correction), c, (L - 1) * c, c


def sig(path, degree, *, time_aug=False, lead_lag=False, end_time=1.0, scalar_term=False, out=None, correction=None):
    """Reference signature_cuda_* on a contiguous CUDA tensor (B, L, d)."""
    import torch
    B, L, d = path.shape
    D = (2 * d if lead_lag else d) + (1 if time_aug else 0)
    n = sum(D ** k for k in range(1, degree + 1)) + (1 if scalar_term else 0)
    if out is None:
        out = torch.empty((B, n), dtype=path.dtype, device=path.device)
    real = _real(path)
    suf = "f" if real is ctypes.c_float else "d"
    rc = getattr(library(), "signature_cuda_" + suf)(_ptr(path), _ptr(out), B, d, L, degree, time_aug, lead_lag,
                                                      real(end_time), True, scalar_term,
                                                      *_correction_args(correction, B, L))
    if rc:
        raise RuntimeError("reference signature_cuda failed with code %d" % rc)
    return out


def sig_backprop(path, sig_, derivs, degree, *, time_aug=False, lead_lag=False, end_time=1.0, scalar_term=False,
                 out=None, correction=None):
    import torch
    B, L, d = path.shape
    if out is None:
        out = torch.empty_like(path)
    real = _real(path)
    suf = "f" if real is ctypes.c_float else "d"
    rc = getattr(library(), "sig_backprop_cuda_" + suf)(_ptr(path), _ptr(out), _ptr(derivs), _ptr(sig_), B, d, L,
                                                         degree, time_aug, lead_lag, real(end_time), scalar_term,
                                                         *_correction_args(correction, B, L))
    if rc:
        raise RuntimeError("reference sig_backprop_cuda failed with code %d" % rc)
    return out


def transform_path(path, *, time_aug=False, lead_lag=False, end_time=1.0):
    """Reference transform_path_cuda_* on a contiguous CUDA tensor (B, L, d)."""
    import torch
    B, L, d = path.shape
    out = torch.empty((B, 2 * L - 1 if lead_lag else L, (2 * d if lead_lag else d) + (1 if time_aug else 0)),
                      dtype=path.dtype, device=path.device)
    real = _real(path)
    suf = "f" if real is ctypes.c_float else "d"
    rc = getattr(library(), "transform_path_cuda_" + suf)(_ptr(path), _ptr(out), B, d, L, time_aug, lead_lag,
                                                           real(end_time))
    if rc:
        raise RuntimeError("reference transform_path_cuda failed with code %d" % rc)
    return out


def transform_path_backprop(derivs, length, dimension, *, time_aug=False, lead_lag=False, end_time=1.0):
    """Reference transform_path_backprop_cuda_*: derivs (B, L', d') -> gradient (B, L, d)."""
    import torch
    B = derivs.shape[0]
    out = torch.empty((B, length, dimension), dtype=derivs.dtype, device=derivs.device)
    real = _real(derivs)
    suf = "f" if real is ctypes.c_float else "d"
    rc = getattr(library(), "transform_path_backprop_cuda_" + suf)(_ptr(derivs), _ptr(out), B, dimension, length,
                                                                    time_aug, lead_lag, real(end_time))
    if rc:
        raise RuntimeError("reference transform_path_backprop_cuda failed with code %d" % rc)
    return out
