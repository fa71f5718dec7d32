"""Shape / dtype / placement handling for the Python operators.

Follows the contract of the reference's handlers (``pysiglib/data_handlers.py:50-260``):
paths are ``(..., L, d)`` with any number of leading batch axes, signatures ``(..., S)``;
NumPy in gives NumPy out, torch in gives torch out on the same device; inputs are made
contiguous and owning before their pointer is taken.  Unlike the reference, host arrays
(NumPy, CPU tensors) are not sent to a CPU library: their pointers go to the same CUDA
entry points, which stage them through the GPU."""
from ctypes import POINTER, cast
from math import prod

import numpy as np
import torch

from .load_cusig import DTYPES
from .param_checks import check_dtype, check_type, own_contiguous


def _describe(arr):
    """(kind, dtype name, device string) of a validated array."""
    if isinstance(arr, np.ndarray):
        return "numpy", str(arr.dtype), "cpu"
    return "torch", str(arr.dtype)[6:], str(arr.device)


def _pointer(arr, dtype):
    if isinstance(arr, np.ndarray):
        return arr.ctypes.data_as(POINTER(DTYPES[dtype]))
    return cast(arr.data_ptr(), POINTER(DTYPES[dtype]))


class PathInput:
    """A path or batch of paths, flattened to (batch, L, d)."""

    def __init__(self, path, time_aug, lead_lag, end_time, name="path"):
        check_type(path, name, (np.ndarray, torch.Tensor))
        self.array = own_contiguous(path)
        check_dtype(self.array, name)
        if self.array.ndim < 2:
            raise ValueError("%s must have at least rank 2, got rank %d." % (name, self.array.ndim))
        self.batch_shape = tuple(self.array.shape[:-2])
        self.batch_size = prod(self.batch_shape) if self.batch_shape else 1
        self.data_length = self.array.shape[-2]
        self.data_dimension = self.array.shape[-1]
        if self.data_dimension == 0:
            raise ValueError("%s has 0 channels (dimension). Path dimension must be at least 1." % name)
        self.kind, self.dtype, self.device = _describe(self.array)
        self.time_aug, self.lead_lag, self.end_time = time_aug, lead_lag, end_time
        self.length = 2 * self.data_length - 1 if lead_lag else self.data_length
        self.dimension = (2 * self.data_dimension if lead_lag else self.data_dimension) + (1 if time_aug else 0)
        self.pointer = _pointer(self.array, self.dtype)


class SigInput:
    """A signature-shaped array ``(..., sig_len)``; a leading scalar term is stripped."""

    def __init__(self, sig, sig_len, name):
        check_type(sig, name, (np.ndarray, torch.Tensor))
        self.array = own_contiguous(sig)
        check_dtype(self.array, name)
        if self.array.ndim < 1:
            raise ValueError("%s must have at least rank 1, got rank 0." % name)
        length = self.array.shape[-1]
        if length == sig_len + 1:
            self.array = own_contiguous(self.array[..., 1:])
            length = sig_len
        if length != sig_len:
            raise ValueError("%s is of incorrect length. Expected %d, got %d" % (name, sig_len, length))
        self.batch_shape = tuple(self.array.shape[:-1])
        self.kind, self.dtype, self.device = _describe(self.array)
        self.pointer = _pointer(self.array, self.dtype)


def check_same(inputs, names):
    """All of kind / dtype / batch shape / device must agree (reference: data_handlers.py:98-128)."""
    joined = ", ".join(names)
    first = inputs[0]
    if any(i.kind != first.kind for i in inputs):
        raise ValueError(joined + " must all be numpy arrays or all torch tensors")
    if any(i.dtype != first.dtype for i in inputs):
        raise ValueError(joined + " must have the same dtype")
    if any(i.batch_shape != first.batch_shape for i in inputs):
        raise ValueError(joined + " have different batch shapes")
    if any(i.device != first.device for i in inputs):
        raise ValueError(joined + " must be on the same device")


class Output:
    """Uninitialised result of shape ``batch_shape + shape`` matching ``like`` in kind, dtype, device."""

    def __init__(self, like, shape):
        full = (*like.batch_shape, *shape)
        if like.kind == "numpy":
            self.array = np.empty(full, dtype=np.float32 if like.dtype == "float32" else np.float64)
        else:
            self.array = torch.empty(full, dtype=torch.float32 if like.dtype == "float32" else torch.float64,
                                     device=like.array.device)
        self.pointer = _pointer(self.array, like.dtype)


class CorrectionInput:
    """Per-segment correction levels of ``sig`` / ``sig_backprop`` (reference:
    ``pysiglib/data_handlers.py:191-260``).  Accepted shapes: ``(C,)`` one correction for every
    segment, ``(L-1, C)`` one per segment shared by the batch, ``batch_shape + (L-1, C)``; ``C``
    must cover tensor levels ``2..k`` of the data dimension for some ``k <= degree``."""

    def __init__(self, correction, path, degree):
        self.array = None
        self.length = 0
        self.pointer = None
        self.batch_stride = 0
        self.segment_stride = 0
        if correction is None:
            return
        check_type(correction, "correction", (np.ndarray, torch.Tensor))
        if isinstance(correction, np.ndarray) != (path.kind == "numpy"):
            raise ValueError("correction must have the same array type as path")
        self.array = own_contiguous(correction)
        check_dtype(self.array, "correction")
        kind, dtype, device = _describe(self.array)
        if dtype != path.dtype:
            raise ValueError("correction and path must have the same dtype")
        if device != path.device:
            raise ValueError("correction and path must be on the same device")
        size = self.array.size if kind == "numpy" else self.array.numel()
        if size == 0:
            return
        if path.lead_lag:
            raise ValueError("correction cannot be used with lead_lag=True")
        shape = tuple(self.array.shape)
        segments = max(path.data_length - 1, 0)
        expected = (*path.batch_shape, segments, shape[-1] if shape else 0)
        message = ("correction shape must be (C,), (path.shape[-2] - 1, C), or " + str(expected) +
                   " for path shape " + str(tuple(path.array.shape)))
        if len(shape) == 0:
            raise ValueError(message)
        if len(shape) == 1:
            self.length = shape[0]
        elif len(shape) == 2 and shape[0] == segments:
            self.length = shape[1]
            self.segment_stride = self.length
        else:
            if shape != expected:
                raise ValueError(message)
            self.length = shape[-1]
            self.batch_stride = segments * self.length
            self.segment_stride = self.length
        if degree < 2:
            raise ValueError("correction must be empty when degree < 2")
        offset, level_size = 0, path.data_dimension
        for _ in range(2, degree + 1):
            level_size *= path.data_dimension
            offset += level_size
            if offset >= self.length:
                break
        if offset != self.length:
            raise ValueError("correction length must be a prefix of tensor levels 2..degree")
        self.pointer = _pointer(self.array, dtype)
