"""Timed CPU baseline (benchmark infrastructure only; never a checker, never the product).

Loads ``libsig_oracle_timing.so``: the oracle's sources compiled like a release build of a CPU
library (``-O3 -march=native``) plus the SIMD-across-paths forward the reference's dispatcher
takes for narrow paths (``siglib/cpsig/cp_signature.h:605-717, 786-804``).  Because the build
is tuned to the machine it runs on, it is compiled on first use on that machine (one gcc run, a
few seconds) into a file named after the CPU's feature flags, not shipped.
"""
import ctypes
import hashlib
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
LANES = {np.dtype(np.float32): 8, np.dtype(np.float64): 4}


def _host_tag():
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags") or line.startswith("model name"):
                    flags += line
                if line.strip() == "" and flags:
                    break
    except OSError:
        pass
    return hashlib.sha256(flags.encode()).hexdigest()[:12]


def library_path():
    return os.path.join(_HERE, "_build", "libsig_oracle_timing.%s.so" % _host_tag())


def build():
    path = library_path()
    sources = [os.path.join(_HERE, f) for f in ("sig_oracle_timing.c", "sig_oracle.c", "sig_oracle_impl.h",
                                                "sig_oracle_algebra.h", "sig_oracle_log.h", "sig_oracle_coef.h")]
    if os.path.exists(path) and all(os.path.getmtime(path) >= os.path.getmtime(s) for s in sources):
        return path
    os.makedirs(os.path.dirname(path), exist_ok=True)
    subprocess.run(["gcc", "-O3", "-march=native", "-fPIC", "-std=c11", "-shared", "-o", path, sources[0], "-lm",
                    "-lpthread"], check=True, capture_output=True, cwd=_HERE)
    return path


def _lib():
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(build())
        u64, ci = ctypes.c_uint64, ctypes.c_int
        for suf, real in (("f", ctypes.c_float), ("d", ctypes.c_double)):
            ptr = ctypes.POINTER(real)
            fn = getattr(lib, "oracle_signature_" + suf)
            fn.restype, fn.argtypes = ci, [ptr, ptr, u64, u64, u64, u64, ci, ci, real, ci, ci, ci]
            fn = getattr(lib, "oracle_sig_backprop_" + suf)
            fn.restype, fn.argtypes = ci, [ptr, ptr, ptr, ptr, u64, u64, u64, u64, ci, ci, real, ci, ci]
            fn = getattr(lib, "oracle_signature_batch_simd_" + suf)
            fn.restype, fn.argtypes = ci, [ptr, ptr, u64, u64, u64, u64, ci, ci]
        _LIB = lib
    return _LIB


def takes_batch_simd(batch, length, dim, degree, dtype):
    """The reference's condition for its SIMD-across-paths forward (cp_signature.h:786-804), for
    calls without flags or corrections."""
    lanes = LANES[np.dtype(dtype)]
    full_len = 1 + sum(dim ** k for k in range(1, degree + 1))
    return degree > 1 and length >= 16 and dim <= 4 and dim < lanes and batch >= lanes and full_len <= 8192


def sig(path, degree, n_threads=1):
    """Forward signature (no flags), the variant the reference's dispatcher would run; returns
    (result, variant name)."""
    path = np.ascontiguousarray(path)
    B, L, d = path.shape
    suf, real = ("f", ctypes.c_float) if path.dtype == np.float32 else ("d", ctypes.c_double)
    ptr = ctypes.POINTER(real)
    n = sum(d ** k for k in range(1, degree + 1))
    out = np.empty((B, n), dtype=path.dtype)
    if takes_batch_simd(B, L, d, degree, path.dtype):
        rc = getattr(_lib(), "oracle_signature_batch_simd_" + suf)(
            path.ctypes.data_as(ptr), out.ctypes.data_as(ptr), B, d, L, degree, 0, int(n_threads))
        variant = "SIMD across paths"
    else:
        rc = getattr(_lib(), "oracle_signature_" + suf)(
            path.ctypes.data_as(ptr), out.ctypes.data_as(ptr), B, d, L, degree, 0, 0, real(1.0), 1, 0, int(n_threads))
        variant = "per-path Horner"
    if rc:
        raise RuntimeError("timing oracle failed with code %d" % rc)
    return out, variant


def sig_backprop(path, sig_, sig_derivs, degree, n_threads=1):
    path = np.ascontiguousarray(path)
    B, L, d = path.shape
    suf, real = ("f", ctypes.c_float) if path.dtype == np.float32 else ("d", ctypes.c_double)
    ptr = ctypes.POINTER(real)
    s2 = np.ascontiguousarray(sig_, dtype=path.dtype)
    g2 = np.ascontiguousarray(sig_derivs, dtype=path.dtype)
    out = np.empty_like(path)
    rc = getattr(_lib(), "oracle_sig_backprop_" + suf)(
        path.ctypes.data_as(ptr), out.ctypes.data_as(ptr), g2.ctypes.data_as(ptr), s2.ctypes.data_as(ptr), B, d, L,
        degree, 0, 0, real(1.0), 0, int(n_threads))
    if rc:
        raise RuntimeError("timing oracle failed with code %d" % rc)
    return out
