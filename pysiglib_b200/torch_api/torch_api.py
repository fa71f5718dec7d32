"""Autograd bridge: ``torch_api.sig`` differentiates through the CUDA signature.

Counterpart of the reference's ``Sig`` Function and ``torch_api.sig``
(``pysiglib/torch_api/torch_api.py:76-117``): the forward saves the path and the
signature itself; the backward calls ``sig_backprop`` on them."""
from typing import Union

import numpy as np
import torch

from ..sig import sig as sig_forward
from ..sig_backprop import sig_backprop


class Sig(torch.autograd.Function):
    @staticmethod
    def forward(ctx, path, correction, degree, time_aug, lead_lag, end_time, horner, scalar_term, n_jobs):
        out = sig_forward(path, degree, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time, horner=horner,
                          scalar_term=scalar_term, correction=correction, n_jobs=n_jobs)
        ctx.save_for_backward(path, out)
        ctx.args = (degree, time_aug, lead_lag, end_time, n_jobs)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        path, out = ctx.saved_tensors
        degree, time_aug, lead_lag, end_time, n_jobs = ctx.args
        grad = sig_backprop(path, out, grad_output, degree, time_aug=time_aug, lead_lag=lead_lag,
                            end_time=end_time, n_jobs=n_jobs)
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
