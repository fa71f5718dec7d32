"""``linear_sig``, ``sig_join`` and ``sig_join_backprop`` on the GPU.

Same names, parameters, validation and result layout as the reference's operators
(``pysiglib/linear_sig.py:28-110``, ``pysiglib/sig_join.py:28-132``,
``pysiglib/sig_join_backprop.py:28-130``); every call goes to the C symbol of the same name in
libcusig.so (``linear_sig_cuda_*``, ``sig_join_cuda_*``, ``sig_join_backprop_cuda_*``)."""
from typing import Union

import numpy as np
import torch

from . import load_cusig
from .data_handlers import Output, check_same
from .error_codes import err_msg
from .param_checks import check_n_jobs, check_non_neg, check_type
from .sig import _Sig, _finish_current_stream
from .sig_length import infer_scalar_term, sig_length


def _vector(arr, length, name):
    v = _Sig(arr, name)
    if v.array.shape[-1] != length:
        raise ValueError("%s is of incorrect length. Expected %d, got %d" % (name, length, v.array.shape[-1]))
    return v


def _check_dims(dimension, degree, n_jobs):
    check_type(dimension, "dimension", int)
    check_non_neg(dimension, "dimension")
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    check_n_jobs(n_jobs)


def linear_sig(
        displacement: Union[np.ndarray, torch.Tensor],
        dimension: int,
        degree: int,
        *,
        scalar_term: bool = False,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Truncated signature of the straight segment from 0 to ``displacement``: level ``k`` is
    ``displacement^(x)k / k!``.

    :param displacement: ``(dimension,)`` or ``(..., dimension)``, float32 / float64.
    :param dimension: number of channels.
    :param degree: truncation level.
    :param scalar_term: include the constant 1 of level 0.
    :param n_jobs: accepted for compatibility.
    """
    _check_dims(dimension, degree, n_jobs)
    check_type(scalar_term, "scalar_term", bool)
    v = _vector(displacement, dimension, "displacement")
    result = Output(v, (sig_length(dimension, degree, scalar_term=scalar_term),))
    if v.batch_size == 0 or result.array.shape[-1] == 0:
        return result.array
    _finish_current_stream(v.array)
    code = load_cusig.fn("linear_sig_cuda", v.dtype)(v.pointer, result.pointer, v.batch_size, dimension, degree,
                                                     scalar_term)
    if code:
        raise Exception("Error in pysiglib.linear_sig: " + err_msg(code))
    return result.array


def sig_join(
        sig: Union[np.ndarray, torch.Tensor],
        displacement: Union[np.ndarray, torch.Tensor],
        dimension: int,
        degree: int,
        *,
        prepend: bool = False,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Extends a signature by one straight segment: ``sig (x) linear_sig(displacement)``, the
    signature of the path followed by that segment; with ``prepend`` the segment comes first,
    ``linear_sig(displacement) (x) sig``.

    :param sig: ``(S,)`` or ``(..., S)``, with or without the scalar term (the result uses the same layout).
    :param displacement: ``(dimension,)`` or ``(..., dimension)`` with the batch shape of ``sig``.
    """
    _check_dims(dimension, degree, n_jobs)
    a = _Sig(sig, "sig")
    scalar_term = infer_scalar_term(a.array, dimension, degree)
    v = _vector(displacement, dimension, "displacement")
    if a.kind != v.kind:
        raise ValueError("sig and displacement must both be numpy arrays or both torch tensors")
    if a.dtype != v.dtype:
        raise ValueError("sig and displacement must have the same dtype")
    if a.batch_shape != v.batch_shape:
        raise ValueError("sig and displacement must have the same batch shape")
    if a.device != v.device:
        raise ValueError("sig and displacement must be on the same device")
    result = Output(a, (a.array.shape[-1],))
    if a.batch_size == 0 or a.array.shape[-1] == 0:
        return result.array
    _finish_current_stream(a.array)
    code = load_cusig.fn("sig_join_cuda", a.dtype)(a.pointer, v.pointer, result.pointer, a.batch_size, dimension,
                                                   degree, bool(prepend), scalar_term)
    if code:
        raise Exception("Error in pysiglib.sig_join: " + err_msg(code))
    return result.array


def sig_join_backprop(
        d_out: Union[np.ndarray, torch.Tensor],
        sig: Union[np.ndarray, torch.Tensor],
        displacement: Union[np.ndarray, torch.Tensor],
        dimension: int,
        degree: int,
        *,
        prepend: bool = False,
        n_jobs: int = 1
):
    """Backward pass of ``sig_join``: from ``dF/d sig_join(sig, displacement)`` to
    ``(dF/d sig, dF/d displacement)``.  ``d_out`` and ``sig`` share one layout; a scalar slot of
    the first result is 0."""
    _check_dims(dimension, degree, n_jobs)
    a = _Sig(sig, "sig")
    scalar_term = infer_scalar_term(a.array, dimension, degree)
    g = _vector(d_out, a.array.shape[-1], "d_out")
    v = _vector(displacement, dimension, "displacement")
    if not (g.kind == a.kind == v.kind):
        raise ValueError("d_out, sig and displacement must all be numpy arrays or all torch tensors")
    if not (g.dtype == a.dtype == v.dtype):
        raise ValueError("d_out, sig and displacement must have the same dtype")
    if not (g.batch_shape == a.batch_shape == v.batch_shape):
        raise ValueError("d_out, sig and displacement must have the same batch shape")
    if not (g.device == a.device == v.device):
        raise ValueError("d_out, sig and displacement must be on the same device")
    d_sig, d_disp = Output(g, (a.array.shape[-1],)), Output(g, (dimension,))
    if g.batch_size == 0:
        return d_sig.array, d_disp.array
    _finish_current_stream(g.array)
    code = load_cusig.fn("sig_join_backprop_cuda", g.dtype)(
        g.pointer, d_sig.pointer, d_disp.pointer, a.pointer, v.pointer, g.batch_size, dimension, degree,
        bool(prepend), scalar_term)
    if code:
        raise Exception("Error in pysiglib.sig_join_backprop: " + err_msg(code))
    return d_sig.array, d_disp.array
