"""Autograd bridge: the functions here differentiate through the CUDA operators.

Counterpart of the reference's autograd Functions (``pysiglib/torch_api/torch_api.py``:
``Sig`` 76-117, ``SigCombine`` 121-153, ``TransformPath`` 206-233, ``SigJoin`` 1182-1212): each
forward saves what its backward needs and the backward calls the matching ``*_backprop``."""
from typing import Union

import numpy as np
import torch

from ..sig import sig as sig_forward
from ..sig import sig_combine as sig_combine_forward
from ..sig import sig_combine_backprop
from ..sig_backprop import sig_backprop
from ..log_sig import sig_to_log_sig as sig_to_log_sig_forward
from ..log_sig import log_sig as log_sig_forward
from ..log_sig import sig_to_log_sig_backprop
from ..sig_coef import sig_coef as sig_coef_forward
from ..sig_coef import sig_coef_backprop
from ..sig_join import sig_join as sig_join_forward
from ..sig_join import sig_join_backprop
from ..transform_path import transform_path as transform_path_forward
from ..transform_path import transform_path_backprop


class Sig(torch.autograd.Function):
    @staticmethod
    def forward(ctx, path, correction, degree, time_aug, lead_lag, end_time, horner, scalar_term, n_jobs):
        out = sig_forward(path, degree, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, horner=horner,
                          scalar_term=scalar_term, correction=correction, n_jobs=n_jobs)
        saved_correction = path.new_empty((0,)) if correction is None else correction.detach().clone()
        ctx.save_for_backward(path, out, saved_correction)
        ctx.args = (degree, time_aug, lead_lag, end_time, n_jobs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        path, out, saved_correction = ctx.saved_tensors
        degree, time_aug, lead_lag, end_time, n_jobs = ctx.args
        correction = saved_correction if saved_correction.numel() != 0 else None
        grad = sig_backprop(path, out, grad_output, degree, time_aug=time_aug, lead_lag=lead_lag,
                            end_time=end_time, correction=correction, n_jobs=n_jobs)
        return (grad,) + (None,) * 8


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
    if not isinstance(path, torch.Tensor):
        return sig_forward(path, degree, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, horner=horner,
                           scalar_term=scalar_term, correction=correction, n_jobs=n_jobs)
    return Sig.apply(path, correction, degree, time_aug, lead_lag, end_time, horner, scalar_term, n_jobs)


sig.__doc__ = sig_forward.__doc__
signature = sig


class SigCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sig1, sig2, dimension, degree, time_aug, lead_lag, n_jobs):
        out = sig_combine_forward(sig1, sig2, dimension, degree, time_aug=time_aug, lead_lag=lead_lag, n_jobs=n_jobs)
        ctx.save_for_backward(sig1, sig2)
        ctx.args = (dimension, degree, time_aug, lead_lag, n_jobs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        sig1, sig2 = ctx.saved_tensors
        dimension, degree, time_aug, lead_lag, n_jobs = ctx.args
        g1, g2 = sig_combine_backprop(grad_output, sig1, sig2, dimension, degree, time_aug=time_aug,
                                      lead_lag=lead_lag, n_jobs=n_jobs)
        return g1, g2, None, None, None, None, None


def sig_combine(sig1, sig2, dimension: int, degree: int, *, time_aug: bool = False, lead_lag: bool = False,
                n_jobs: int = 1):
    if not isinstance(sig1, torch.Tensor):
        return sig_combine_forward(sig1, sig2, dimension, degree, time_aug=time_aug, lead_lag=lead_lag, n_jobs=n_jobs)
    return SigCombine.apply(sig1, sig2, dimension, degree, time_aug, lead_lag, n_jobs)


sig_combine.__doc__ = sig_combine_forward.__doc__


class SigJoin(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sig_, displacement, dimension, degree, prepend, n_jobs):
        out = sig_join_forward(sig_, displacement, dimension, degree, prepend=bool(prepend), n_jobs=n_jobs)
        ctx.save_for_backward(sig_, displacement)
        ctx.args = (dimension, degree, bool(prepend), n_jobs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        sig_, displacement = ctx.saved_tensors
        dimension, degree, prepend, n_jobs = ctx.args
        d_sig, d_disp = sig_join_backprop(grad_output, sig_, displacement, dimension, degree, prepend=prepend,
                                          n_jobs=n_jobs)
        return d_sig, d_disp, None, None, None, None


def sig_join(sig, displacement, dimension: int, degree: int, *, prepend: bool = False, n_jobs: int = 1):
    if not isinstance(sig, torch.Tensor):
        return sig_join_forward(sig, displacement, dimension, degree, prepend=prepend, n_jobs=n_jobs)
    return SigJoin.apply(sig, displacement, dimension, degree, int(prepend), n_jobs)


sig_join.__doc__ = sig_join_forward.__doc__


class TransformPath(torch.autograd.Function):
    @staticmethod
    def forward(ctx, path, time_aug, lead_lag, end_time, n_jobs):
        out = transform_path_forward(path, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, n_jobs=n_jobs)
        ctx.args = (time_aug, lead_lag, end_time, n_jobs)
        return out.clone() if out is path else out

    @staticmethod
    def backward(ctx, grad_output):
        time_aug, lead_lag, end_time, n_jobs = ctx.args
        grad = transform_path_backprop(grad_output, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time,
                                       n_jobs=n_jobs)
        return grad, None, None, None, None


def transform_path(path, *, time_aug: bool = False, lead_lag: bool = False, end_time: float = 1., n_jobs: int = 1):
    if not isinstance(path, torch.Tensor):
        return transform_path_forward(path, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, n_jobs=n_jobs)
    return TransformPath.apply(path, time_aug, lead_lag, end_time, n_jobs)


transform_path.__doc__ = transform_path_forward.__doc__


class SigToLogSig(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sig_, dimension, degree, time_aug, lead_lag, method, n_jobs):
        out = sig_to_log_sig_forward(sig_, dimension, degree, time_aug=time_aug, lead_lag=lead_lag, method=method,
                                     n_jobs=n_jobs)
        ctx.save_for_backward(sig_)
        ctx.args = (dimension, degree, time_aug, lead_lag, method, n_jobs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        dimension, degree, time_aug, lead_lag, method, n_jobs = ctx.args
        grad = sig_to_log_sig_backprop(ctx.saved_tensors[0], grad_output, dimension, degree, time_aug=time_aug,
                                       lead_lag=lead_lag, method=method, n_jobs=n_jobs)
        return grad, None, None, None, None, None, None


def sig_to_log_sig(sig, dimension: int, degree: int, *, time_aug: bool = False, lead_lag: bool = False,
                   method: int = 1, n_jobs: int = 1):
    if not isinstance(sig, torch.Tensor):
        return sig_to_log_sig_forward(sig, dimension, degree, time_aug=time_aug, lead_lag=lead_lag, method=method,
                                      n_jobs=n_jobs)
    return SigToLogSig.apply(sig, dimension, degree, time_aug, lead_lag, method, n_jobs)


sig_to_log_sig.__doc__ = sig_to_log_sig_forward.__doc__


def log_sig(path, degree: int, *, time_aug: bool = False, lead_lag: bool = False, end_time: float = 1.,
            method: int = 1, scalar_term: bool = False, correction=None, n_jobs: int = 1):
    if not isinstance(path, torch.Tensor):
        return log_sig_forward(path, degree, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, method=method,
                               scalar_term=scalar_term, correction=correction, n_jobs=n_jobs)
    sig_ = sig(path, degree, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, scalar_term=scalar_term,
               correction=correction, n_jobs=n_jobs)
    return sig_to_log_sig(sig_, path.shape[-1], degree, time_aug=time_aug, lead_lag=lead_lag, method=method,
                          n_jobs=n_jobs)


log_sig.__doc__ = log_sig_forward.__doc__


def _coef_from_prefixes(words, coef, prefixes):
    """The forward always computes all prefixes (the backward needs them); keep the last of each word."""
    if prefixes:
        return coef
    if isinstance(words, tuple):
        words = [words]
    last, pos = [], 0
    for w in words:
        pos += max(len(w), 1)
        last.append(pos - 1)
    return coef[..., last].contiguous()


class SigCoef(torch.autograd.Function):
    @staticmethod
    def forward(ctx, path, words, time_aug, lead_lag, end_time, n_jobs):
        coefs = sig_coef_forward(path, words, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, prefixes=True,
                                 n_jobs=n_jobs)
        ctx.save_for_backward(coefs, path)
        ctx.args = (words, time_aug, lead_lag, end_time, n_jobs)
        return coefs

    @staticmethod
    def backward(ctx, grad_output):
        coefs, path = ctx.saved_tensors
        words, time_aug, lead_lag, end_time, n_jobs = ctx.args
        grad = sig_coef_backprop(path, words, coefs, grad_output, time_aug=time_aug, lead_lag=lead_lag,
                                 end_time=end_time, n_jobs=n_jobs)
        return grad, None, None, None, None, None


def sig_coef(path, words, *, time_aug: bool = False, lead_lag: bool = False, end_time: float = 1.,
             prefixes: bool = False, n_jobs: int = 1):
    if not isinstance(path, torch.Tensor):
        return sig_coef_forward(path, words, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time,
                                prefixes=prefixes, n_jobs=n_jobs)
    return _coef_from_prefixes(words, SigCoef.apply(path, words, time_aug, lead_lag, end_time, n_jobs), prefixes)


sig_coef.__doc__ = sig_coef_forward.__doc__
