"""``sig``: truncated signature of a path or a batch of paths, computed on a B200.

Python surface of the reference's ``pysiglib.sig`` (``pysiglib/sig.py:128-312``): same
parameters, defaults, type checks, error texts and result layout."""
import ctypes
import warnings
from typing import Union

import numpy as np
import torch

from . import load_cusig
from .data_handlers import CorrectionInput, Output, PathInput, SigInput, check_same
from .error_codes import err_msg
from .param_checks import check_n_jobs, check_non_neg, check_type
from .sig_length import infer_scalar_term, sig_length

NONFINITE_WARNING = ("sig produced NaN or Inf values. This is typically caused by paths with large "
                     "increments, leading to numerical overflow. Consider normalizing your paths.")


def _current_stream(array):
    if isinstance(array, torch.Tensor) and array.is_cuda:
        return ctypes.c_void_p(torch.cuda.current_stream(array.device).cuda_stream)
    return ctypes.c_void_p(None)


def _finish_current_stream(*arrays):
    """For the entry points that keep the reference's signature (no stream argument): they run on
    the legacy default stream, which is not ordered after work queued on a non-blocking side
    stream (every torch side stream is one).  If the caller's current stream on a tensor's device
    is such a stream, wait for it, so the kernels never read an operand that is still being
    produced; the calls themselves return only when their result is complete."""
    seen = set()
    for array in arrays:
        if isinstance(array, torch.Tensor) and array.is_cuda and array.device not in seen:
            seen.add(array.device)
            stream = torch.cuda.current_stream(array.device)
            if stream.cuda_stream != 0:
                stream.synchronize()


def sig(
        path: Union[np.ndarray, torch.Tensor],
        degree: int,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        end_time: float = 1.,
        horner: bool = True,
        scalar_term: bool = False,
        correction=None,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Truncated signature of ``path`` up to level ``degree``.

    ``path`` has shape ``(length, dimension)`` or ``(..., length, dimension)``; the result has
    shape ``(..., S)`` with ``S = sum_{k=1..degree} D^k`` where ``D`` is the dimension after the
    optional transforms.  Level ``k`` occupies ``D^k`` consecutive entries; inside a level the
    coefficient of the word ``(i_1, .., i_k)`` sits at ``i_1 D^(k-1) + .. + i_k``.

    :param path: ``numpy.ndarray`` or ``torch.Tensor`` of dtype float32 / float64.  CUDA tensors
        are processed in place on their device; NumPy arrays and CPU tensors are streamed
        through the current CUDA device and the result is returned on the host.
    :param degree: truncation level, a non-negative ``int``.
    :param time_aug: append time as a last channel, running from 0 to ``end_time``.
    :param lead_lag: apply the lead-lag transform (``2*length - 1`` points, channels
        ``[lag, lead]``) before taking the signature.
    :param end_time: final time of the time channel (``float``).
    :param horner: accepted for compatibility; the Horner scheme is always used.
    :param scalar_term: include the constant 1 of level 0 as the first entry.
    :param correction: optional higher-level terms added to every segment's logarithm: the segment
        from ``x_j`` to ``x_{j+1}`` contributes ``exp((x_{j+1} - x_j) + c_j)`` with ``c_j`` living on
        tensor levels ``2..k`` (``k <= degree``) of the path's own channels.  Shape ``(C,)`` (the same
        for every segment), ``(length - 1, C)`` or ``batch_shape + (length - 1, C)`` with
        ``C = d^2 + .. + d^k``.  Not available with ``lead_lag``.
    :param n_jobs: accepted for compatibility (validated, otherwise ignored on the GPU).
    :return: array of the same kind, dtype and device as ``path``.

    A ``RuntimeWarning`` is issued when the result contains NaN or Inf.

    Example::

        import torch, pysiglib_b200
        x = torch.rand(32, 100, 5, device="cuda")
        s = pysiglib_b200.sig(x, 4)            # (32, 780)
    """
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    check_type(horner, "horner", bool)
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_type(end_time, "end_time", float)
    check_type(scalar_term, "scalar_term", bool)
    check_n_jobs(n_jobs)

    data = PathInput(path, time_aug, lead_lag, end_time)
    corr = CorrectionInput(correction, data, degree)
    n = sig_length(data.dimension, degree, scalar_term=scalar_term)
    result = Output(data, (n,))
    if data.batch_size == 0:
        return result.array

    if corr.length:
        # the reference's own symbol carries the correction arguments (synchronous)
        _finish_current_stream(data.array)
        code = load_cusig.fn("signature_cuda", data.dtype)(
            data.pointer, result.pointer, data.batch_size, data.data_dimension, data.data_length, degree,
            time_aug, lead_lag, end_time, horner, scalar_term, corr.pointer, corr.length, corr.batch_stride,
            corr.segment_stride)
        if code:
            raise Exception("Error in pysiglib.sig: " + err_msg(code))
        finite = np.isfinite(result.array).all() if data.kind == "numpy" else bool(torch.isfinite(result.array).all())
        if not finite:
            warnings.warn(NONFINITE_WARNING, RuntimeWarning, stacklevel=2)
        return result.array

    bad = ctypes.c_int(0)
    code = load_cusig.fn("sigb200_signature", data.dtype)(
        data.pointer, result.pointer, data.batch_size, data.data_dimension, data.data_length, degree,
        time_aug, lead_lag, end_time, scalar_term, _current_stream(data.array), 1, ctypes.byref(bad))
    if code:
        raise Exception("Error in pysiglib.sig: " + err_msg(code))
    if bad.value:
        warnings.warn(NONFINITE_WARNING, RuntimeWarning, stacklevel=2)
    return result.array


signature = sig


class _Sig:
    """A signature-shaped input kept in the caller's layout (a scalar term is not stripped)."""

    def __init__(self, arr, name):
        from .data_handlers import _describe, _pointer
        from .param_checks import check_dtype, own_contiguous
        check_type(arr, name, (np.ndarray, torch.Tensor))
        self.array = own_contiguous(arr)
        check_dtype(self.array, name)
        if self.array.ndim < 1:
            raise ValueError("%s must have at least rank 1, got rank 0." % name)
        self.batch_shape = tuple(self.array.shape[:-1])
        self.kind, self.dtype, self.device = _describe(self.array)
        self.pointer = _pointer(self.array, self.dtype)

    @property
    def batch_size(self):
        n = 1
        for extent in self.batch_shape:
            n *= extent
        return n


def sig_combine(
        sig1: Union[np.ndarray, torch.Tensor],
        sig2: Union[np.ndarray, torch.Tensor],
        dimension: int,
        degree: int,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Signature of a concatenated path from the signatures of its two parts (Chen's identity).

    If ``sig1 = sig(x1)`` and ``sig2 = sig(x2)`` where ``x2`` starts where ``x1`` ends, the
    result is ``sig(x1 * x2) = sig1 (x) sig2`` truncated at ``degree``.  Same parameters as the
    reference's ``pysiglib.sig_combine`` (``pysiglib/sig.py:28-126``).

    :param sig1, sig2: arrays ``(..., S)`` of the same kind, dtype, device and batch shape, both
        with or both without the scalar term (the result uses the same layout).
    :param dimension: dimension of the underlying path (before ``time_aug`` / ``lead_lag``).
    :param degree: truncation level of both signatures.
    :param time_aug, lead_lag: the flags the signatures were computed with (they only change the
        effective dimension).
    :param n_jobs: accepted for compatibility.
    """
    check_type(dimension, "dimension", int)
    check_type(degree, "degree", int)
    check_non_neg(dimension, "dimension")
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_n_jobs(n_jobs)
    a, b = _Sig(sig1, "sig1"), _Sig(sig2, "sig2")
    scalar_term = infer_scalar_term(a.array, dimension, degree, time_aug=time_aug, lead_lag=lead_lag)
    if b.array.shape[-1] != a.array.shape[-1]:
        raise ValueError("sig2 is of incorrect length. Expected %d, got %d" % (a.array.shape[-1], b.array.shape[-1]))
    check_same([a, b], ["sig1", "sig2"])
    result = Output(a, (a.array.shape[-1],))
    batch = a.batch_size
    if batch == 0 or a.array.shape[-1] == 0:
        return result.array
    from .sig_length import aug_dim
    _finish_current_stream(a.array)
    code = load_cusig.fn("sig_combine_cuda", a.dtype)(
        a.pointer, b.pointer, result.pointer, batch, aug_dim(dimension, time_aug, lead_lag), degree, scalar_term)
    if code:
        raise Exception("Error in pysiglib.sig_combine: " + err_msg(code))
    return result.array


def sig_combine_backprop(
        deriv: Union[np.ndarray, torch.Tensor],
        sig1: Union[np.ndarray, torch.Tensor],
        sig2: Union[np.ndarray, torch.Tensor],
        dimension: int,
        degree: int,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        n_jobs: int = 1
):
    """Backward pass of ``sig_combine``: from ``dF/d sig_combine(sig1, sig2)`` to
    ``(dF/d sig1, dF/d sig2)``.  Same parameters as the reference's
    ``pysiglib.sig_combine_backprop`` (``pysiglib/sig_backprop.py:27-126``); all three inputs
    share one layout (with or without the scalar term) and the results use it too, with zeros
    in the scalar slots.
    """
    check_type(dimension, "dimension", int)
    check_type(degree, "degree", int)
    check_non_neg(dimension, "dimension")
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_n_jobs(n_jobs)
    d, a, b = _Sig(deriv, "deriv"), _Sig(sig1, "sig1"), _Sig(sig2, "sig2")
    scalar_term = infer_scalar_term(a.array, dimension, degree, time_aug=time_aug, lead_lag=lead_lag)
    for other, name in ((b, "sig2"), (d, "deriv")):
        if other.array.shape[-1] != a.array.shape[-1]:
            raise ValueError("%s is of incorrect length. Expected %d, got %d"
                             % (name, a.array.shape[-1], other.array.shape[-1]))
    check_same([d, a, b], ["deriv", "sig1", "sig2"])
    out1, out2 = Output(a, (a.array.shape[-1],)), Output(a, (a.array.shape[-1],))
    if a.batch_size == 0 or a.array.shape[-1] == 0:
        return out1.array, out2.array
    from .sig_length import aug_dim
    _finish_current_stream(a.array)
    code = load_cusig.fn("sig_combine_backprop_cuda", a.dtype)(
        d.pointer, out1.pointer, out2.pointer, a.pointer, b.pointer, a.batch_size,
        aug_dim(dimension, time_aug, lead_lag), degree, scalar_term)
    if code:
        raise Exception("Error in pysiglib.sig_combine_backprop: " + err_msg(code))
    return out1.array, out2.array
