"""Argument validation shared by the Python operators.

Same rules and exception types as the reference (``pysiglib/param_checks.py:28-104``):
wrong Python types raise TypeError, bad values ValueError; arrays that are views, have a
zero stride or are not C-contiguous are copied once, with a warning the first time."""
import warnings

import numpy as np
import torch

SUPPORTED_DTYPES = (np.float32, np.float64, torch.float32, torch.float64)


def _type_name(t):
    return getattr(t, "__name__", str(t))


def check_type(value, name, type_):
    types = type_ if isinstance(type_, tuple) else (type_,)
    if not isinstance(value, types):
        wanted = " or ".join(_type_name(t) for t in types)
        raise TypeError("%s must be of type %s, got %s instead" % (name, wanted, _type_name(type(value))))


def check_non_neg(value, name):
    if value < 0:
        raise ValueError("%s must be a non-negative integer, got %s = %s" % (name, name, value))


def check_n_jobs(n_jobs):
    check_type(n_jobs, "n_jobs", int)
    if n_jobs == 0:
        raise ValueError("n_jobs cannot be 0")


def check_dtype(arr, name):
    if arr.dtype not in SUPPORTED_DTYPES:
        raise TypeError("%s.dtype must be float or double, got %s instead" % (name, arr.dtype))


_warned_about_copy = False
COPY_WARNING = ("Received an array that is a view, has a zero stride or is not contiguous; it is copied "
                "before use. Pass a contiguous array that owns its data to avoid the copy. "
                "This warning is shown once per session.")


def own_contiguous(arr):
    """Return ``arr`` if it is contiguous and owns its storage, else a contiguous copy."""
    global _warned_about_copy
    if isinstance(arr, torch.Tensor):
        needs_copy = arr._base is not None or not arr.is_contiguous() or any(s == 0 for s in arr.stride())
        copy = (lambda: arr.clone().contiguous())
    elif isinstance(arr, np.ndarray):
        needs_copy = arr.base is not None or not arr.flags["C_CONTIGUOUS"]
        copy = (lambda: np.ascontiguousarray(arr.copy()))
    else:
        raise TypeError("expected a numpy.ndarray or torch.Tensor")
    if not needs_copy:
        return arr
    if not _warned_about_copy:
        warnings.warn(COPY_WARNING, stacklevel=4)
        _warned_about_copy = True
    return copy()
