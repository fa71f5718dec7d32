"""``transform_path`` and ``transform_path_backprop`` on the GPU.

Same names, parameters and layout as the reference's operators
(``pysiglib/transform_path.py:28-153``, ``pysiglib/transform_path_backprop.py:28-107``); the calls
go to ``transform_path_cuda_*`` / ``transform_path_backprop_cuda_*`` in libcusig.so."""
from typing import Union

import numpy as np
import torch

from . import load_cusig
from .data_handlers import Output, PathInput
from .error_codes import err_msg
from .param_checks import check_n_jobs, check_type
from .sig import _finish_current_stream


def transform_path(
        path: Union[np.ndarray, torch.Tensor],
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        end_time: float = 1.,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Materialises the transformed path the signature operators see.

    ``lead_lag`` turns ``(..., L, d)`` into ``(..., 2L-1, 2d)`` with channels ``[lag, lead]`` (the
    lead moves first); ``time_aug`` appends a channel running linearly from 0 to ``end_time``.
    With neither flag the input is returned unchanged."""
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_type(end_time, "end_time", float)
    if not time_aug and not lead_lag:
        return path
    check_n_jobs(n_jobs)
    data = PathInput(path, time_aug, lead_lag, end_time)
    if time_aug and data.data_length < 2:
        raise ValueError("transform_path(time_aug=True) requires path length >= 2, got %d. " % data.data_length)
    result = Output(data, (data.length, data.dimension))
    if data.batch_size == 0:
        return result.array
    _finish_current_stream(data.array)
    code = load_cusig.fn("transform_path_cuda", data.dtype)(
        data.pointer, result.pointer, data.batch_size, data.data_dimension, data.data_length, time_aug, lead_lag,
        end_time)
    if code:
        raise Exception("Error in pysiglib.transform_path: " + err_msg(code))
    return result.array


def transform_path_backprop(
        derivs: Union[np.ndarray, torch.Tensor],
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        end_time: float = 1.,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Backward pass of ``transform_path``: derivatives with respect to the transformed path
    ``(..., L', d')`` in, derivatives with respect to the original path ``(..., L, d)`` out."""
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_type(end_time, "end_time", float)
    if not time_aug and not lead_lag:
        return derivs
    check_n_jobs(n_jobs)
    data = PathInput(derivs, False, False, end_time, "derivs")
    length = (data.length + 1) // 2 if lead_lag else data.length
    dimension = data.dimension - 1 if time_aug else data.dimension
    if lead_lag:
        dimension //= 2
    result = Output(data, (length, dimension))
    if data.batch_size == 0 or length == 0 or dimension == 0:
        return result.array
    _finish_current_stream(data.array)
    code = load_cusig.fn("transform_path_backprop_cuda", data.dtype)(
        data.pointer, result.pointer, data.batch_size, dimension, length, time_aug, lead_lag, end_time)
    if code:
        raise Exception("Error in pysiglib.transform_path_backprop: " + err_msg(code))
    return result.array
