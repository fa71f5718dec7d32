"""ctypes front-end of the CPU oracle (test infrastructure only).

The oracle restates pySigLib's CPU arithmetic for ``sig`` and ``sig_backprop``
(see ``sig_oracle_impl.h`` for the reference file:line map).  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libsig_oracle.so")
_LIB = None


def build(force=False):
    """Compile the oracle with gcc (idempotent)."""
    src = [os.path.join(_HERE, f) for f in ("sig_oracle.c", "sig_oracle_impl.h", "sig_oracle_algebra.h", "sig_oracle_log.h", "sig_oracle_coef.h")]
    if (not force and os.path.exists(_LIB_PATH)
            and all(os.path.getmtime(_LIB_PATH) >= os.path.getmtime(s) for s in src)):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


def _lib():
    global _LIB
    if _LIB is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        u64 = ctypes.c_uint64
        for suf, real in (("f", ctypes.c_float), ("d", ctypes.c_double)):
            ptr = ctypes.POINTER(real)
            fwd = getattr(lib, "oracle_signature_" + suf)
            fwd.restype = ctypes.c_int
            fwd.argtypes = [ptr, ptr, u64, u64, u64, u64, ctypes.c_int, ctypes.c_int, real,
                            ctypes.c_int, ctypes.c_int, ctypes.c_int]
            bwd = getattr(lib, "oracle_sig_backprop_" + suf)
            bwd.restype = ctypes.c_int
            bwd.argtypes = [ptr, ptr, ptr, ptr, u64, u64, u64, u64, ctypes.c_int, ctypes.c_int,
                            real, ctypes.c_int, ctypes.c_int]
            cmb = getattr(lib, "oracle_sig_combine_" + suf)
            cmb.restype = ctypes.c_int
            cmb.argtypes = [ptr, ptr, ptr, u64, u64, u64, ctypes.c_int]
            cbp = getattr(lib, "oracle_sig_combine_backprop_" + suf)
            cbp.restype = ctypes.c_int
            cbp.argtypes = [ptr, ptr, ptr, ptr, ptr, u64, u64, u64, ctypes.c_int]
            ci = ctypes.c_int
            for name, args in (
                    ("oracle_signature_correction_", [ptr, ptr, u64, u64, u64, u64, ci, real, ci, ptr, u64, u64, u64]),
                    ("oracle_sig_backprop_correction_",
                     [ptr, ptr, ptr, ptr, u64, u64, u64, u64, ci, real, ci, ptr, u64, u64, u64]),
                    ("oracle_tensor_exp_", [ptr, ptr, u64, u64]),
                    ("oracle_tensor_exp_backprop_", [ptr, ptr, ptr, u64, u64]),
                    ("oracle_sig_to_log_sig_", [ptr, ptr, u64, u64, u64, ci, ci]),
                    ("oracle_sig_to_log_sig_backprop_", [ptr, ptr, ptr, u64, u64, u64, ci, ci]),
                    ("oracle_sig_coef_", [ptr, ptr, ctypes.POINTER(u64), u64, ctypes.POINTER(u64), u64, u64, u64, ci, ci,
                                          real, ci]),
                    ("oracle_sig_coef_backprop_", [ptr, ptr, ptr, ptr, ctypes.POINTER(u64), u64, ctypes.POINTER(u64),
                                                   u64, u64, u64, ci, ci, real]),
                    ("oracle_linear_sig_", [ptr, ptr, u64, u64, u64, ci]),
                    ("oracle_sig_join_", [ptr, ptr, ptr, u64, u64, u64, ci, ci]),
                    ("oracle_sig_join_backprop_", [ptr, ptr, ptr, ptr, ptr, u64, u64, u64, ci, ci])):
                fn = getattr(lib, name + suf)
                fn.restype = ctypes.c_int
                fn.argtypes = args
        lib.oracle_lyndon_indices.restype = u64
        lib.oracle_lyndon_indices.argtypes = [u64, u64, ctypes.POINTER(u64), u64]
        lib.oracle_sig_length.restype = u64
        lib.oracle_sig_length.argtypes = [u64, u64]
        _LIB = lib
    return _LIB


def _suffix(arr):
    if arr.dtype == np.float32:
        return "f", ctypes.c_float
    if arr.dtype == np.float64:
        return "d", ctypes.c_double
    raise TypeError("oracle supports float32 / float64 only")


def aug_dim(d, time_aug, lead_lag):
    return (2 * d if lead_lag else d) + (1 if time_aug else 0)


def sig_length(dim, degree, scalar_term=False):
    n = _lib().oracle_sig_length(dim, degree)
    return n - (0 if scalar_term else 1)


def _correction_layout(correction, B, L, dtype):
    """(array, length, batch stride, segment stride) for the three accepted shapes: (C,),
    (L-1, C) and (B, L-1, C) (pysiglib/data_handlers.py:233-258)."""
    c = np.ascontiguousarray(correction, dtype=dtype)
    if c.ndim == 1:
        return c, c.shape[0], 0, 0
    if c.ndim == 2 and c.shape[0] == max(L - 1, 0):
        return c, c.shape[1], 0, c.shape[1]
    if c.shape[:-1] != (B, max(L - 1, 0)):
        raise ValueError("correction shape")
    return c, c.shape[-1], max(L - 1, 0) * c.shape[-1], c.shape[-1]


def sig(path, degree, *, time_aug=False, lead_lag=False, end_time=1.0, horner=True,
        scalar_term=False, n_threads=1, correction=None):
    """Oracle signature of ``path`` (B, L, d) or (L, d); numpy in, numpy out.  ``correction``
    adds per-segment higher-level terms: segment signature = exp(increment + correction)."""
    path = np.ascontiguousarray(path)
    single = path.ndim == 2
    p3 = path[None] if single else path
    B, L, d = p3.shape
    suf, real = _suffix(p3)
    n = sig_length(aug_dim(d, time_aug, lead_lag), degree, scalar_term)
    out = np.empty((B, n), dtype=p3.dtype)
    ptr = ctypes.POINTER(real)
    if correction is not None and np.size(correction):
        if lead_lag:
            raise ValueError("correction cannot be used with lead_lag")
        c, clen, bs, ss = _correction_layout(correction, B, L, p3.dtype)
        rc = getattr(_lib(), "oracle_signature_correction_" + suf)(
            p3.ctypes.data_as(ptr), out.ctypes.data_as(ptr), B, d, L, degree, int(time_aug), real(end_time),
            int(scalar_term), c.ctypes.data_as(ptr), clen, bs, ss)
        if rc:
            raise RuntimeError("oracle_signature_correction failed with code %d" % rc)
        return out[0] if single else out
    rc = getattr(_lib(), "oracle_signature_" + suf)(
        p3.ctypes.data_as(ptr), out.ctypes.data_as(ptr), B, d, L, degree,
        int(time_aug), int(lead_lag), real(end_time), int(horner), int(scalar_term), int(n_threads))
    if rc:
        raise RuntimeError("oracle_signature failed with code %d" % rc)
    return out[0] if single else out


def sig_backprop(path, sig_, sig_derivs, degree, *, time_aug=False, lead_lag=False,
                 end_time=1.0, n_threads=1, correction=None):
    """Oracle gradient of sum(sig * sig_derivs) w.r.t. ``path``; scalar-term format inferred."""
    path = np.ascontiguousarray(path)
    single = path.ndim == 2
    p3 = path[None] if single else path
    B, L, d = p3.shape
    suf, real = _suffix(p3)
    full = sig_length(aug_dim(d, time_aug, lead_lag), degree, True)
    s2 = np.ascontiguousarray(sig_, dtype=p3.dtype).reshape(B, -1)
    g2 = np.ascontiguousarray(sig_derivs, dtype=p3.dtype).reshape(B, -1)
    if s2.shape[1] not in (full, full - 1) or g2.shape != s2.shape:
        raise ValueError("sig / sig_derivs have the wrong length")
    scalar_term = s2.shape[1] == full
    out = np.empty_like(p3)
    ptr = ctypes.POINTER(real)
    if correction is not None and np.size(correction):
        if lead_lag:
            raise ValueError("correction cannot be used with lead_lag")
        c, clen, bs, ss = _correction_layout(correction, B, L, p3.dtype)
        rc = getattr(_lib(), "oracle_sig_backprop_correction_" + suf)(
            p3.ctypes.data_as(ptr), out.ctypes.data_as(ptr), g2.ctypes.data_as(ptr), s2.ctypes.data_as(ptr),
            B, d, L, degree, int(time_aug), real(end_time), int(scalar_term), c.ctypes.data_as(ptr), clen, bs, ss)
        if rc:
            raise RuntimeError("oracle_sig_backprop_correction failed with code %d" % rc)
        return out[0] if single else out
    rc = getattr(_lib(), "oracle_sig_backprop_" + suf)(
        p3.ctypes.data_as(ptr), out.ctypes.data_as(ptr), g2.ctypes.data_as(ptr),
        s2.ctypes.data_as(ptr), B, d, L, degree, int(time_aug), int(lead_lag), real(end_time),
        int(scalar_term), int(n_threads))
    if rc:
        raise RuntimeError("oracle_sig_backprop failed with code %d" % rc)
    return out[0] if single else out


def sig_combine(sig1, sig2, dim, degree):
    """Oracle Chen product of two (batches of) signatures of a ``dim``-channel path; the
    scalar-term layout is inferred from the length."""
    a = np.ascontiguousarray(sig1)
    single = a.ndim == 1
    a2 = a[None] if single else a.reshape(-1, a.shape[-1])
    b2 = np.ascontiguousarray(sig2, dtype=a.dtype).reshape(a2.shape)
    suf, real = _suffix(a2)
    full = sig_length(dim, degree, True)
    if a2.shape[1] not in (full, full - 1):
        raise ValueError("signatures have the wrong length")
    out = np.empty_like(a2)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_sig_combine_" + suf)(a2.ctypes.data_as(ptr), b2.ctypes.data_as(ptr),
                                                      out.ctypes.data_as(ptr), a2.shape[0], dim, degree,
                                                      int(a2.shape[1] == full))
    if rc:
        raise RuntimeError("oracle_sig_combine failed with code %d" % rc)
    return out[0] if single else out.reshape(a.shape)


def sig_combine_backprop(deriv, sig1, sig2, dim, degree):
    """Oracle adjoints (d sig1, d sig2) of sig_combine; scalar-term layout inferred from the length."""
    a = np.ascontiguousarray(sig1)
    a2 = a.reshape(-1, a.shape[-1])
    b2 = np.ascontiguousarray(sig2, dtype=a.dtype).reshape(a2.shape)
    d2 = np.ascontiguousarray(deriv, dtype=a.dtype).reshape(a2.shape)
    suf, real = _suffix(a2)
    full = sig_length(dim, degree, True)
    if a2.shape[1] not in (full, full - 1):
        raise ValueError("signatures have the wrong length")
    o1, o2 = np.empty_like(a2), np.empty_like(a2)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_sig_combine_backprop_" + suf)(
        d2.ctypes.data_as(ptr), o1.ctypes.data_as(ptr), o2.ctypes.data_as(ptr), a2.ctypes.data_as(ptr),
        b2.ctypes.data_as(ptr), a2.shape[0], dim, degree, int(a2.shape[1] == full))
    if rc:
        raise RuntimeError("oracle_sig_combine_backprop failed with code %d" % rc)
    return o1.reshape(a.shape), o2.reshape(a.shape)


def tensor_exp(log_sig, dim, degree):
    """Oracle truncated tensor exponential of one element given WITH its scalar slot (ignored)."""
    x = np.ascontiguousarray(log_sig)
    suf, real = _suffix(x)
    out = np.empty_like(x)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_tensor_exp_" + suf)(x.ctypes.data_as(ptr), out.ctypes.data_as(ptr), dim, degree)
    if rc:
        raise RuntimeError("oracle_tensor_exp failed with code %d" % rc)
    return out


def tensor_exp_backprop(d_sig, log_sig, dim, degree):
    """Oracle adjoint of tensor_exp (both arrays with their scalar slots)."""
    x = np.ascontiguousarray(log_sig)
    g = np.ascontiguousarray(d_sig, dtype=x.dtype)
    suf, real = _suffix(x)
    out = np.empty_like(x)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_tensor_exp_backprop_" + suf)(out.ctypes.data_as(ptr), g.ctypes.data_as(ptr),
                                                              x.ctypes.data_as(ptr), dim, degree)
    if rc:
        raise RuntimeError("oracle_tensor_exp_backprop failed with code %d" % rc)
    return out


def linear_sig(displacement, degree, scalar_term=False):
    """Oracle signature of the straight segment with the given displacement(s) (..., d)."""
    v = np.ascontiguousarray(displacement)
    v2 = v.reshape(-1, v.shape[-1])
    suf, real = _suffix(v2)
    dim = v2.shape[1]
    out = np.empty((v2.shape[0], sig_length(dim, degree, scalar_term)), dtype=v2.dtype)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_linear_sig_" + suf)(v2.ctypes.data_as(ptr), out.ctypes.data_as(ptr), v2.shape[0],
                                                     dim, degree, int(scalar_term))
    if rc:
        raise RuntimeError("oracle_linear_sig failed with code %d" % rc)
    return out.reshape(v.shape[:-1] + (out.shape[1],))


def sig_join(sig_, displacement, dim, degree, prepend=False):
    """Oracle sig (x) linear_sig(displacement) (or the reverse product with prepend=True)."""
    a = np.ascontiguousarray(sig_)
    a2 = a.reshape(-1, a.shape[-1])
    v2 = np.ascontiguousarray(displacement, dtype=a.dtype).reshape(a2.shape[0], dim)
    suf, real = _suffix(a2)
    full = sig_length(dim, degree, True)
    if a2.shape[1] not in (full, full - 1):
        raise ValueError("signature has the wrong length")
    out = np.empty_like(a2)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_sig_join_" + suf)(a2.ctypes.data_as(ptr), v2.ctypes.data_as(ptr),
                                                   out.ctypes.data_as(ptr), a2.shape[0], dim, degree, int(prepend),
                                                   int(a2.shape[1] == full))
    if rc:
        raise RuntimeError("oracle_sig_join failed with code %d" % rc)
    return out.reshape(a.shape)


def sig_join_backprop(d_out, sig_, displacement, dim, degree, prepend=False):
    """Oracle adjoints (d sig, d displacement) of sig_join."""
    a = np.ascontiguousarray(sig_)
    a2 = a.reshape(-1, a.shape[-1])
    v = np.ascontiguousarray(displacement, dtype=a.dtype)
    v2 = v.reshape(a2.shape[0], dim)
    g2 = np.ascontiguousarray(d_out, dtype=a.dtype).reshape(a2.shape)
    suf, real = _suffix(a2)
    full = sig_length(dim, degree, True)
    if a2.shape[1] not in (full, full - 1):
        raise ValueError("signature has the wrong length")
    d_sig, d_disp = np.empty_like(a2), np.empty_like(v2)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_sig_join_backprop_" + suf)(
        g2.ctypes.data_as(ptr), d_sig.ctypes.data_as(ptr), d_disp.ctypes.data_as(ptr), a2.ctypes.data_as(ptr),
        v2.ctypes.data_as(ptr), a2.shape[0], dim, degree, int(prepend), int(a2.shape[1] == full))
    if rc:
        raise RuntimeError("oracle_sig_join_backprop failed with code %d" % rc)
    return d_sig.reshape(a.shape), d_disp.reshape(v.shape)


def lyndon_indices(dim, degree):
    """Flat positions (scalar slot = 0) of the Lyndon words of length <= degree, by length then
    lexicographically: the coordinates log-signature method 1 keeps."""
    n = _lib().oracle_lyndon_indices(dim, degree, None, 0)
    out = np.zeros(n, dtype=np.uint64)
    _lib().oracle_lyndon_indices(dim, degree, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), n)
    return out


def log_sig_length(dim, degree):
    return int(_lib().oracle_lyndon_indices(dim, degree, None, 0))


def lyndon_words(dim, degree):
    """Lyndon words of length 1..degree over ``dim`` letters, by length then lexicographically
    (Duval's algorithm; the order of siglib/shared/preparation/log_sig/lyndon_words.cpp:25-84)."""
    out = []
    for n in range(1, degree + 1):
        w = [0]
        while w:
            m = len(w)
            if m == n:
                out.append(tuple(w))
            while len(w) < n:
                w.append(w[len(w) - m])
            while w and w[-1] == dim - 1:
                w.pop()
            if w:
                w[-1] += 1
    return out


def lyndon_bracket_expansions(dim, degree):
    """For every Lyndon word w (in lyndon_words order) the expansion of its bracket [w] into words:
    a dict {word: integer coefficient}; [w] = [[u], [v]] with v the longest proper Lyndon suffix
    (standard factorisation, lyndon_words.cpp:114-138, 181-232)."""
    words = lyndon_words(dim, degree)
    index = {w: i for i, w in enumerate(words)}
    exps = []
    for w in words:
        if len(w) == 1:
            exps.append({w: 1})
            continue
        cut = next(i for i in range(1, len(w)) if w[i:] in index)
        eu, ev = exps[index[w[:cut]]], exps[index[w[cut:]]]
        e = {}
        for a, ca in eu.items():
            for b, cb in ev.items():
                e[a + b] = e.get(a + b, 0) + ca * cb
                e[b + a] = e.get(b + a, 0) - ca * cb
        exps.append({k: v for k, v in e.items() if v})
    return words, exps


def lyndon_projection(dim, degree):
    """P[i][j] = coefficient of the Lyndon word w_i in the bracket [w_j]: Lyndon-word coordinates
    of a Lie element are P times its Lyndon-basis coordinates (method 1 = P @ method 2)."""
    words, exps = lyndon_bracket_expansions(dim, degree)
    index = {w: i for i, w in enumerate(words)}
    P = np.zeros((len(words), len(words)))
    for j, e in enumerate(exps):
        for w, c in e.items():
            if w in index:
                P[index[w], j] = c
    return P


def sig_to_log_sig(sig_, dim, degree, method=1):
    """Oracle log signature from (batches of) signatures; method 0 = expanded tensor logarithm in
    the layout of the input, method 1 = its coordinates at the Lyndon words, method 2 = its
    coordinates in the Lyndon (bracket) basis, P^-1 applied to method 1 as the reference does
    (siglib/cpsig/cp_tensor_log.h:160-170)."""
    if method == 2:
        words = sig_to_log_sig(sig_, dim, degree, method=1)
        return np.linalg.solve(lyndon_projection(dim, degree), words.reshape(-1, words.shape[-1]).T.astype(np.float64)
                               ).T.reshape(words.shape).astype(words.dtype)
    a = np.ascontiguousarray(sig_)
    a2 = a.reshape(-1, a.shape[-1])
    suf, real = _suffix(a2)
    full = sig_length(dim, degree, True)
    if a2.shape[1] not in (full, full - 1):
        raise ValueError("signature has the wrong length")
    n_out = a2.shape[1] if method == 0 else log_sig_length(dim, degree)
    out = np.empty((a2.shape[0], n_out), dtype=a2.dtype)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_sig_to_log_sig_" + suf)(a2.ctypes.data_as(ptr), out.ctypes.data_as(ptr), a2.shape[0],
                                                         dim, degree, method, int(a2.shape[1] == full))
    if rc:
        raise RuntimeError("oracle_sig_to_log_sig failed with code %d" % rc)
    return out.reshape(a.shape[:-1] + (n_out,))


def sig_to_log_sig_backprop(sig_, log_sig_derivs, dim, degree, method=1):
    """Oracle dF/d sig from dF/d log_sig (layouts as in sig_to_log_sig)."""
    if method == 2:  # cp_tensor_log.h:261-283: transpose of P^-1, then the Lyndon-word backward
        g = np.asarray(log_sig_derivs)
        pulled = np.linalg.solve(lyndon_projection(dim, degree).T, g.reshape(-1, g.shape[-1]).T.astype(np.float64)
                                 ).T.reshape(g.shape).astype(g.dtype)
        return sig_to_log_sig_backprop(sig_, pulled, dim, degree, method=1)
    a = np.ascontiguousarray(sig_)
    a2 = a.reshape(-1, a.shape[-1])
    g2 = np.ascontiguousarray(log_sig_derivs, dtype=a.dtype).reshape(a2.shape[0], -1)
    suf, real = _suffix(a2)
    full = sig_length(dim, degree, True)
    out = np.empty_like(a2)
    ptr = ctypes.POINTER(real)
    rc = getattr(_lib(), "oracle_sig_to_log_sig_backprop_" + suf)(
        a2.ctypes.data_as(ptr), out.ctypes.data_as(ptr), g2.ctypes.data_as(ptr), a2.shape[0], dim, degree, method,
        int(a2.shape[1] == full))
    if rc:
        raise RuntimeError("oracle_sig_to_log_sig_backprop failed with code %d" % rc)
    return out.reshape(a.shape)


def _words(words):
    words = [words] if isinstance(words, tuple) else list(words)
    flat = np.array([i for w in words for i in w] + [0], dtype=np.uint64)
    degrees = np.array([len(w) for w in words] + [0], dtype=np.uint64)
    return words, flat, degrees


def sig_coef(path, words, *, time_aug=False, lead_lag=False, end_time=1.0, prefixes=False):
    """Oracle signature coefficients of ``path`` (B, L, d) or (L, d) at the given word(s)."""
    path = np.ascontiguousarray(path)
    single = path.ndim == 2
    p3 = path[None] if single else path
    B, L, d = p3.shape
    suf, real = _suffix(p3)
    words, flat, degrees = _words(words)
    n_out = sum((len(w) if (prefixes and w) else 1) for w in words)
    out = np.empty((B, n_out), dtype=p3.dtype)
    ptr, u64p = ctypes.POINTER(real), ctypes.POINTER(ctypes.c_uint64)
    rc = getattr(_lib(), "oracle_sig_coef_" + suf)(
        p3.ctypes.data_as(ptr), out.ctypes.data_as(ptr), flat.ctypes.data_as(u64p), len(words),
        degrees.ctypes.data_as(u64p), B, d, L, int(time_aug), int(lead_lag), real(end_time), int(prefixes))
    if rc:
        raise RuntimeError("oracle_sig_coef failed with code %d" % rc)
    return out[0] if single else out


def sig_coef_backprop(path, words, coefs, derivs, *, time_aug=False, lead_lag=False, end_time=1.0):
    """Oracle gradient w.r.t. the path; ``coefs`` / ``derivs`` in the prefixes=True layout."""
    path = np.ascontiguousarray(path)
    single = path.ndim == 2
    p3 = path[None] if single else path
    B, L, d = p3.shape
    suf, real = _suffix(p3)
    words, flat, degrees = _words(words)
    c2 = np.ascontiguousarray(coefs, dtype=p3.dtype).reshape(B, -1)
    g2 = np.ascontiguousarray(derivs, dtype=p3.dtype).reshape(B, -1)
    out = np.empty_like(p3)
    ptr, u64p = ctypes.POINTER(real), ctypes.POINTER(ctypes.c_uint64)
    rc = getattr(_lib(), "oracle_sig_coef_backprop_" + suf)(
        p3.ctypes.data_as(ptr), out.ctypes.data_as(ptr), c2.ctypes.data_as(ptr), g2.ctypes.data_as(ptr),
        flat.ctypes.data_as(u64p), len(words), degrees.ctypes.data_as(u64p), B, d, L, int(time_aug), int(lead_lag),
        real(end_time))
    if rc:
        raise RuntimeError("oracle_sig_coef_backprop failed with code %d" % rc)
    return out[0] if single else out
