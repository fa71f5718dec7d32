"""``sig_to_log_sig``, its backward pass, and ``log_sig`` on the GPU, methods 0, 1 and 2.

Same names, parameters and layouts as the reference's operators (``pysiglib/log_sig.py:95-188,
241-329, 331-470``, ``pysiglib/log_sig_backprop.py:30-137``):

* method 0: the expanded tensor logarithm, in the layout of the signature (scalar slot 0);
* method 1: its coordinates at the Lyndon words, ``log_sig_length`` values;
* method 2: its coordinates in the Lyndon (bracket) basis, ``log_sig_length`` values.

Method 3 (from the path, without the signature) is not part of this build and raises
``NotImplementedError``."""
import ctypes
import warnings
from typing import Union

import numpy as np
import torch

from . import load_cusig
from .data_handlers import Output, PathInput
from .error_codes import err_msg
from .param_checks import check_n_jobs, check_non_neg, check_type
from .sig import NONFINITE_WARNING, _Sig, _current_stream, _finish_current_stream, sig
from .sig_length import aug_dim, infer_scalar_term, log_sig_length, sig_length


def _check_method(method, where):
    check_type(method, "method", int)
    if method < 0 or method > 3:
        raise ValueError("method must be one of 0, 1, 2 or 3. Got " + str(method) + " instead.")
    if method == 3 and where != "log_sig":
        raise ValueError("method=3 is not supported in %s. Use log_sig(path, degree, method=3) instead." % where)
    if method == 3:
        raise NotImplementedError("log-signature method 3 is not part of pysiglib_b200 (methods 0, 1 and 2 are)")


def prepare_log_sig(dimension: int, degree: int, method: int, *, time_aug: bool = False, lead_lag: bool = False,
                    use_disk: bool = False, device: str = "both"):
    """Builds what ``method`` needs ahead of time (optional here: method 0 needs nothing; the table of
    Lyndon-word positions of methods 1 and 2 and the inverse projection matrix of method 2 are
    otherwise built at the first call on each GPU)."""
    check_type(dimension, "dimension", int)
    check_non_neg(dimension, "dimension")
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    _check_method(method, "log_sig")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    if method == 0:
        return
    code = load_cusig.library().prepare_log_sig_cuda(aug_dim(dimension, time_aug, lead_lag), degree, method,
                                                     bool(use_disk))
    if code:
        raise Exception("Error in pysiglib.prepare_log_sig: " + err_msg(code))


def sig_to_log_sig(
        sig: Union[np.ndarray, torch.Tensor],
        dimension: int,
        degree: int,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        method: int = 1,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Log signature from the signature.

    :param sig: ``(..., S)`` with or without the scalar term (inferred from the length).
    :param dimension: dimension of the underlying path, before ``time_aug`` / ``lead_lag``.
    :param method: 0 = expanded (result in the layout of ``sig``), 1 = Lyndon-word coordinates,
        2 = Lyndon-basis coordinates (``log_sig_length`` values each).
    """
    check_type(dimension, "dimension", int)
    check_non_neg(dimension, "dimension")
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    _check_method(method, "sig_to_log_sig")
    d = aug_dim(dimension, time_aug, lead_lag)
    a = _Sig(sig, "sig")
    scalar_term = infer_scalar_term(a.array, dimension, degree, time_aug=time_aug, lead_lag=lead_lag)
    out_len = log_sig_length(d, degree) if method else a.array.shape[-1]
    result = Output(a, (out_len,))
    if a.batch_size == 0:
        return result.array
    check_n_jobs(n_jobs)
    _finish_current_stream(a.array)
    code = load_cusig.fn("sig_to_log_sig_cuda", a.dtype)(a.pointer, result.pointer, a.batch_size, d, degree, method,
                                                         scalar_term)
    if code:
        raise Exception("Error in pysiglib.sig_to_log_sig: " + err_msg(code))
    return result.array


def sig_to_log_sig_backprop(
        sig: Union[np.ndarray, torch.Tensor],
        log_sig_derivs: Union[np.ndarray, torch.Tensor],
        dimension: int,
        degree: int,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        method: int = 1,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Backward pass of ``sig_to_log_sig``: ``dF/d log_sig`` (layout of the forward's result) in,
    ``dF/d sig`` (layout of ``sig``, scalar slot 0) out."""
    check_type(dimension, "dimension", int)
    check_non_neg(dimension, "dimension")
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    _check_method(method, "sig_to_log_sig_backprop")
    d = aug_dim(dimension, time_aug, lead_lag)
    a = _Sig(sig, "sig")
    scalar_term = infer_scalar_term(a.array, dimension, degree, time_aug=time_aug, lead_lag=lead_lag)
    g = _Sig(log_sig_derivs, "log_sig_derivs")
    expected = log_sig_length(d, degree) if method else a.array.shape[-1]
    if g.array.shape[-1] != expected:
        raise ValueError("log_sig_derivs is of incorrect length. Expected %d, got %d" % (expected, g.array.shape[-1]))
    if a.kind != g.kind:
        raise ValueError("sig and log_sig_derivs must both be numpy arrays or both torch tensors")
    if a.dtype != g.dtype:
        raise ValueError("sig and log_sig_derivs must have the same dtype")
    if a.batch_shape != g.batch_shape:
        raise ValueError("sig and log_sig_derivs have different batch shapes")
    if a.device != g.device:
        raise ValueError("sig and log_sig_derivs must be on the same device")
    result = Output(a, (a.array.shape[-1],))
    if a.batch_size == 0:
        return result.array
    check_n_jobs(n_jobs)
    _finish_current_stream(a.array)
    code = load_cusig.fn("sig_to_log_sig_backprop_cuda", a.dtype)(a.pointer, result.pointer, g.pointer, a.batch_size, d,
                                                                  degree, method, scalar_term)
    if code:
        raise Exception("Error in pysiglib.sig_to_log_sig_backprop: " + err_msg(code))
    return result.array


def log_sig(
        path: Union[np.ndarray, torch.Tensor],
        degree: int,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        end_time: float = 1.,
        method: int = 1,
        scalar_term: bool = False,
        correction=None,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Log signature of a path (methods 0, 1 and 2): the reference composes ``sig`` and
    ``sig_to_log_sig`` in Python (``pysiglib/log_sig.py:457``); here it is ONE native call in which the
    signature is never written to an array the caller sees, and for shapes with a fused kernel never
    leaves the GPU's SMs at all.  ``scalar_term`` only matters for method 0, whose result has the layout
    of the signature.  With a ``correction`` the two-step composition is used.

    A ``RuntimeWarning`` is issued when the underlying signature contains NaN or Inf, as ``sig`` does."""
    _check_method(method, "log_sig")
    has_correction = correction is not None and (
        correction.numel() if isinstance(correction, torch.Tensor) else np.size(correction)) > 0
    if has_correction:
        sig_ = sig(path, degree, scalar_term=scalar_term, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time,
                   horner=True, correction=correction, n_jobs=n_jobs)
        return sig_to_log_sig(sig_, path.shape[-1], degree, time_aug=time_aug, lead_lag=lead_lag, method=method,
                              n_jobs=n_jobs)
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_type(end_time, "end_time", float)
    check_type(scalar_term, "scalar_term", bool)
    check_n_jobs(n_jobs)
    data = PathInput(path, time_aug, lead_lag, end_time)
    out_len = log_sig_length(data.dimension, degree) if method else sig_length(data.dimension, degree,
                                                                               scalar_term=scalar_term)
    result = Output(data, (out_len,))
    if data.batch_size == 0:
        return result.array
    bad = ctypes.c_int(0)
    code = load_cusig.fn("sigb200_log_sig", data.dtype)(
        data.pointer, result.pointer, data.batch_size, data.data_dimension, data.data_length, degree, time_aug, lead_lag,
        end_time, method, scalar_term, _current_stream(data.array), 1, ctypes.byref(bad))
    if code:
        raise Exception("Error in pysiglib.log_sig: " + err_msg(code))
    if bad.value:
        warnings.warn(NONFINITE_WARNING, RuntimeWarning, stacklevel=2)
    return result.array
