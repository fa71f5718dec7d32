"""Single-box batch partitioner: one call, the batch sharded over several B200s.

The signature of every path is independent, forward and backward, so the batch is cut
into contiguous slices (remainder to the first devices), each device works on its slice
with its own streams, and nothing is exchanged between devices.  The reference has no
multi-GPU path; this module is the new layer between the Python operators and the C ABI.

Host arrays (NumPy / CPU tensors) go through the C-side partitioner
(``sigb200_signature_sharded_*``: one host thread per device, copies overlapped with
compute).  Lists of CUDA tensors already resident on different devices are processed
concurrently on each tensor's own device and stream."""
import ctypes

import numpy as np
import torch

from . import load_cusig
from .data_handlers import Output, PathInput, SigInput, check_same
from .error_codes import err_msg
from .param_checks import check_non_neg, check_type
from .sig_length import infer_scalar_term, sig_length


def shard_bounds(batch_size, n_shards):
    """[(begin, end)] of contiguous shards; the first ``batch_size % n_shards`` get one extra."""
    n = max(1, min(n_shards, max(batch_size, 1)))
    chunk, rem = divmod(batch_size, n)
    bounds, begin = [], 0
    for g in range(n):
        end = begin + chunk + (1 if g < rem else 0)
        bounds.append((begin, end))
        begin = end
    return bounds


def _device_array(devices):
    if devices is None:
        return None, torch.cuda.device_count()
    arr = (ctypes.c_int * len(devices))(*[int(d) for d in devices])
    return arr, len(devices)


def sig_sharded(path, degree, *, devices=None, time_aug=False, lead_lag=False, end_time=1., scalar_term=False):
    """``sig`` of a host-resident batch computed on several GPUs; returns a host array."""
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    data = PathInput(path, time_aug, lead_lag, end_time)
    if data.device != "cpu":
        raise ValueError("sig_sharded takes host arrays; for CUDA tensors call sig on each device's shard")
    result = Output(data, (sig_length(data.dimension, degree, scalar_term=scalar_term),))
    if data.batch_size == 0:
        return result.array
    dev, n = _device_array(devices)
    code = load_cusig.fn("sigb200_signature_sharded", data.dtype)(
        data.pointer, result.pointer, data.batch_size, data.data_dimension, data.data_length, degree,
        time_aug, lead_lag, end_time, scalar_term, dev, n)
    if code:
        raise Exception("Error in pysiglib.sig: " + err_msg(code))
    return result.array


def sig_backprop_sharded(path, sig, sig_derivs, degree, *, devices=None, time_aug=False, lead_lag=False,
                         end_time=1.):
    """``sig_backprop`` of a host-resident batch computed on several GPUs."""
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    data = PathInput(path, time_aug, lead_lag, end_time)
    if data.device != "cpu":
        raise ValueError("sig_backprop_sharded takes host arrays")
    infer_scalar_term(sig, data.data_dimension, degree, time_aug=time_aug, lead_lag=lead_lag)
    n_sig = sig_length(data.dimension, degree, scalar_term=False)
    sig_in, der_in = SigInput(sig, n_sig, "sig"), SigInput(sig_derivs, n_sig, "sig_derivs")
    check_same([sig_in, der_in], ["sig", "sig_derivs"])
    if data.kind != sig_in.kind or data.dtype != sig_in.dtype or data.batch_shape != sig_in.batch_shape:
        raise ValueError("path, sig and sig_derivs must agree in array type, dtype and batch shape")
    result = Output(data, (data.data_length, data.data_dimension))
    if data.batch_size == 0:
        return result.array
    dev, n = _device_array(devices)
    code = load_cusig.fn("sigb200_sig_backprop_sharded", data.dtype)(
        data.pointer, result.pointer, der_in.pointer, sig_in.pointer, data.batch_size, data.data_dimension,
        data.data_length, degree, time_aug, lead_lag, end_time, False, dev, n)
    if code:
        raise Exception("Error in pysiglib.sig_backprop: " + err_msg(code))
    return result.array
