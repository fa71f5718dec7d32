"""``sig_backprop``: gradient of a scalar loss through ``sig``, computed on a B200.

Python surface of the reference's ``pysiglib.sig_backprop``
(``pysiglib/sig_backprop.py:128-256``)."""
from typing import Union

import numpy as np
import torch

from . import load_cusig
from .data_handlers import CorrectionInput, Output, PathInput, SigInput, check_same
from .error_codes import err_msg
from .param_checks import check_n_jobs, check_non_neg, check_type
from .sig import _current_stream, _finish_current_stream
from .sig_length import infer_scalar_term, sig_length


def sig_backprop(
        path: Union[np.ndarray, torch.Tensor],
        sig: Union[np.ndarray, torch.Tensor],
        sig_derivs: Union[np.ndarray, torch.Tensor],
        degree: int,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        end_time: float = 1.,
        correction=None,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Derivative of a scalar ``F`` with respect to ``path``, given ``dF/d sig(path)``.

    :param path: the path(s) the signature was taken of, ``(..., length, dimension)``.
    :param sig: ``sig(path, degree, ...)`` with the same flags, with or without the scalar
        term (inferred from its last axis).  The backward sweep starts from it and rebuilds
        the intermediate signatures by multiplying with inverse increments, so nothing else
        from the forward pass is needed.
    :param sig_derivs: ``dF/d sig``, same shape as ``sig`` (the scalar slot, if present, is ignored).
    :param degree: truncation level used for ``sig``.
    :param time_aug, lead_lag, end_time: the flags used for ``sig``.
    :param correction: the correction ``sig`` was computed with (same shapes as there); the result is
        still the gradient with respect to the path only.
    :param n_jobs: accepted for compatibility.
    :return: ``dF/d path`` with the shape, kind, dtype and device of ``path``.

    Example::

        s = pysiglib_b200.sig(x, 4)
        g = pysiglib_b200.sig_backprop(x, s, torch.ones_like(s), 4)
    """
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_type(end_time, "end_time", float)

    data = PathInput(path, time_aug, lead_lag, end_time)
    corr = CorrectionInput(correction, data, degree)
    check_type(sig, "sig", (np.ndarray, torch.Tensor))
    scalar_term = infer_scalar_term(sig, data.data_dimension, degree, time_aug=time_aug, lead_lag=lead_lag)
    n = sig_length(data.dimension, degree, scalar_term=False)
    sig_in = SigInput(sig, n, "sig")
    der_in = SigInput(sig_derivs, n, "sig_derivs")
    check_same([sig_in, der_in], ["sig", "sig_derivs"])
    if data.kind != sig_in.kind:
        raise ValueError("path, sig and sig_derivs must all be numpy arrays or torch tensors")
    if data.dtype != sig_in.dtype:
        raise ValueError("path, sig and sig_derivs must have the same dtype")
    result = Output(data, (data.data_length, data.data_dimension))
    if data.batch_size == 0:
        return result.array
    if data.batch_shape != sig_in.batch_shape:
        raise ValueError("path, sig and sig_derivs must have the same batch shape")
    if data.device != sig_in.device:
        raise ValueError("path, sig and sig_derivs must be on the same device")
    check_n_jobs(n_jobs)
    del scalar_term  # SigInput has already stripped the scalar slot

    if corr.length:
        _finish_current_stream(data.array)
        code = load_cusig.fn("sig_backprop_cuda", data.dtype)(
            data.pointer, result.pointer, der_in.pointer, sig_in.pointer, data.batch_size, data.data_dimension,
            data.data_length, degree, time_aug, lead_lag, end_time, False, corr.pointer, corr.length,
            corr.batch_stride, corr.segment_stride)
        if code:
            raise Exception("Error in pysiglib.sig_backprop: " + err_msg(code))
        return result.array

    code = load_cusig.fn("sigb200_sig_backprop", data.dtype)(
        data.pointer, result.pointer, der_in.pointer, sig_in.pointer, data.batch_size, data.data_dimension,
        data.data_length, degree, time_aug, lead_lag, end_time, False, _current_stream(data.array), 1)
    if code:
        raise Exception("Error in pysiglib.sig_backprop: " + err_msg(code))
    return result.array
