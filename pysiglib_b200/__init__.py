"""pysiglib_b200: pySigLib's ``sig`` / ``sig_backprop`` path on NVIDIA B200 (sm_100a), with the
operators either side of it (``sig_combine``, ``sig_join``, ``linear_sig``, ``transform_path``, ``sig_coef``, ``sig_to_log_sig`` / ``log_sig`` methods 0, 1 and 2).

Drop-in for that path only: the functions below keep the reference's names, parameters
and result layout, and the shared library keeps the reference's C entry points.  All
computation runs in hand-written CUDA kernels; there is no CPU implementation."""
from .sig import sig, sig_combine, sig_combine_backprop, signature
from .sig_backprop import sig_backprop
from .sig_coef import extract_sig_coef, sig_coef, sig_coef_backprop
from .sig_join import linear_sig, sig_join, sig_join_backprop
from .transform_path import transform_path, transform_path_backprop
from .sig_length import log_sig_length, sig_length
from .log_sig import log_sig, prepare_log_sig, sig_to_log_sig, sig_to_log_sig_backprop
from .sharded import all_gather_signatures, sig_backprop_sharded, sig_multi_device, sig_sharded
from . import torch_api

__version__ = "0.1.0"
__all__ = ["sig", "signature", "sig_combine", "sig_combine_backprop", "sig_backprop", "sig_coef", "sig_coef_backprop", "extract_sig_coef", "sig_join", "sig_join_backprop", "linear_sig", "transform_path", "transform_path_backprop", "sig_length", "log_sig_length", "log_sig", "sig_to_log_sig", "sig_to_log_sig_backprop", "prepare_log_sig", "sig_sharded", "sig_backprop_sharded", "sig_multi_device", "all_gather_signatures", "torch_api"]
