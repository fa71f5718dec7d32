"""``sig_coef``, ``sig_coef_backprop`` and ``extract_sig_coef`` on the GPU.

Same names, parameters and layouts as the reference's operators (``pysiglib/sig_coef.py:29-261``,
``pysiglib/sig_coef_backprop.py:29-189``).  As in the reference's CUDA path, ``time_aug`` /
``lead_lag`` are applied by materialising the transformed path first (and pulling the gradient
back through ``transform_path_backprop``); the kernels see plain paths."""
import ctypes
from typing import Union

import numpy as np
import torch

from . import load_cusig
from .data_handlers import Output, PathInput
from .error_codes import err_msg
from .param_checks import check_n_jobs, check_non_neg, check_type
from .sig import _Sig, _finish_current_stream
from .sig_length import aug_dim
from .transform_path import transform_path, transform_path_backprop


def _check_word(word, max_val, name):
    if not isinstance(word, tuple):
        raise TypeError(name + " must be a tuple of integers.")
    for i in word:
        if not isinstance(i, int) or isinstance(i, bool):
            raise TypeError(name + " must be a tuple of integers.")
        if i < 0 or i >= max_val:
            raise ValueError(name + " must consist of integers in the range [0, " + str(max_val - 1) + "]")


def check_word_or_word_list(words, max_val, name):
    """A word (tuple of ints in [0, max_val)) or a list of words; returns a list of words."""
    try:
        if isinstance(words, tuple):
            _check_word(words, max_val, name)
            return [words]
        if isinstance(words, list):
            for w in words:
                _check_word(w, max_val, "Every word in " + name)
            return words
    except Exception as e:
        raise type(e)("Error processing words: " + str(e)) from e
    raise TypeError(name + " must be a tuple of integers or a list of tuples of integers.")


def word_to_idx(word, dimension, *, scalar_term=False):
    """Position of ``word`` in a flat signature of a ``dimension``-channel path."""
    if not word and not scalar_term:
        raise ValueError("The empty word has no index with scalar_term=False")
    idx = 0
    for letter in word:
        idx = idx * dimension + letter + 1
    return idx if scalar_term else idx - 1


def _word_arrays(words, like):
    """uint64 letter / length arrays where ``like`` lives, and pointers to them."""
    flat = [i for w in words for i in w]
    degrees = [len(w) for w in words]
    if like.kind == "numpy" or like.device == "cpu":
        a, b = np.array(flat + [0], dtype=np.uint64), np.array(degrees + [0], dtype=np.uint64)
        ptrs = (a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)), b.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64)))
    else:
        a = torch.tensor(flat + [0], dtype=torch.uint64, device=like.array.device)
        b = torch.tensor(degrees + [0], dtype=torch.uint64, device=like.array.device)
        ptrs = (ctypes.cast(a.data_ptr(), ctypes.POINTER(ctypes.c_uint64)),
                ctypes.cast(b.data_ptr(), ctypes.POINTER(ctypes.c_uint64)))
    return (a, b), ptrs


def extract_sig_coef(sig, words, dimension: int, *, time_aug: bool = False, lead_lag: bool = False,
                     scalar_term: bool = False):
    """Picks the coefficients at ``words`` out of a signature (or batch) ``(..., S)``."""
    check_type(dimension, "dimension", int)
    check_non_neg(dimension, "dimension")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    d = aug_dim(dimension, time_aug, lead_lag)
    words = check_word_or_word_list(words, d, "word")
    _Sig(sig, "sig")
    return sig[..., [word_to_idx(w, d, scalar_term=scalar_term) for w in words]]


def sig_coef(
        path: Union[np.ndarray, torch.Tensor],
        words,
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        end_time: float = 1.,
        prefixes: bool = False,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Signature coefficients of ``path`` at the given word(s) only.

    :param words: a tuple of channel indices or a list of such tuples; indices refer to the channels
        after ``lead_lag`` / ``time_aug``.
    :param prefixes: also return the coefficients of every proper prefix of each word (they come for
        free): ``[(1, 2), (3, 2, 1)]`` yields the values for ``(1,), (1, 2), (3,), (3, 2), (3, 2, 1)``.
    :return: ``(..., number of requested coefficients)``.
    """
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_type(end_time, "end_time", float)
    check_type(prefixes, "prefixes", bool)
    data = PathInput(path, time_aug, lead_lag, end_time)
    if time_aug or lead_lag:
        transformed = transform_path(path, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time)
        return sig_coef(transformed, words, prefixes=prefixes, n_jobs=n_jobs)
    words = check_word_or_word_list(words, data.dimension, "word")
    if len(words) == 0:
        raise ValueError("words must be a non-empty list of multi-indices.")
    if any(len(w) > 32 for w in words):
        raise ValueError("words longer than 32 letters are not supported")
    result_length = sum((len(w) if (prefixes and w) else 1) for w in words)
    result = Output(data, (result_length,))
    if data.batch_size == 0:
        return result.array
    check_n_jobs(n_jobs)
    keep, (idx_ptr, deg_ptr) = _word_arrays(words, data)
    _finish_current_stream(data.array)
    code = load_cusig.fn("sig_coef_cuda", data.dtype)(
        data.pointer, result.pointer, idx_ptr, len(words), deg_ptr, data.batch_size, data.data_dimension,
        data.data_length, prefixes)
    del keep
    if code:
        raise Exception("Error in pysiglib.sig_coef: " + err_msg(code))
    return result.array


def sig_coef_backprop(
        path: Union[np.ndarray, torch.Tensor],
        words,
        coefs: Union[np.ndarray, torch.Tensor],
        derivs: Union[np.ndarray, torch.Tensor],
        *,
        time_aug: bool = False,
        lead_lag: bool = False,
        end_time: float = 1.,
        n_jobs: int = 1
) -> Union[np.ndarray, torch.Tensor]:
    """Backward pass of ``sig_coef``: ``coefs`` is the forward result computed with ``prefixes=True``,
    ``derivs`` the derivatives of the loss with respect to those values; returns the derivatives with
    respect to ``path``."""
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    check_type(end_time, "end_time", float)
    data = PathInput(path, time_aug, lead_lag, end_time)
    if time_aug or lead_lag:
        transformed = transform_path(path, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time)
        aug_grad = sig_coef_backprop(transformed, words, coefs, derivs, n_jobs=n_jobs)
        return transform_path_backprop(aug_grad, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time)
    words = check_word_or_word_list(words, data.dimension, "word")
    if any(len(w) > 32 for w in words):
        raise ValueError("words longer than 32 letters are not supported")
    coefs_len = sum((len(w) if w else 1) for w in words)
    if coefs.shape[-1] != coefs_len:
        raise ValueError("Expected coefs.shape[-1] == " + str(coefs_len) +
                         ". Please make sure coefs was generated using prefixes=True.")
    c, g = _Sig(coefs, "coef"), _Sig(derivs, "deriv")
    if g.array.shape[-1] != coefs_len:
        raise ValueError("deriv is of incorrect length. Expected %d, got %d" % (coefs_len, g.array.shape[-1]))
    for other, name in ((c, "coef"), (g, "deriv")):
        if other.kind != data.kind:
            raise ValueError("path, coef and deriv must all be numpy arrays or all torch tensors")
        if other.dtype != data.dtype:
            raise ValueError("path, coef and deriv must have the same dtype")
        if other.batch_shape != data.batch_shape:
            raise ValueError("path, coef and deriv have different batch shapes")
        if other.device != data.device:
            raise ValueError("path, coef and deriv must be on the same device")
    result = Output(data, (data.data_length, data.data_dimension))
    if data.batch_size == 0:
        return result.array
    check_n_jobs(n_jobs)
    keep, (idx_ptr, deg_ptr) = _word_arrays(words, data)
    _finish_current_stream(data.array)
    code = load_cusig.fn("sig_coef_backprop_cuda", data.dtype)(
        data.pointer, result.pointer, c.pointer, g.pointer, idx_ptr, len(words), deg_ptr, data.batch_size,
        data.data_dimension, data.data_length)
    del keep
    if code:
        raise Exception("Error in pysiglib.sig_coef_backprop: " + err_msg(code))
    return result.array
