"""Differentiable front-end (same names as the base package, no ``*_backprop``)."""
from ..sig_length import sig_length
from .torch_api import (Sig, SigCoef, SigCombine, SigJoin, SigToLogSig, TransformPath, log_sig, sig, sig_coef,
                        sig_combine, sig_join, sig_to_log_sig, signature, transform_path)

__all__ = ["sig", "signature", "sig_combine", "sig_join", "transform_path", "log_sig", "sig_to_log_sig", "sig_coef", "sig_length", "Sig", "SigCoef", "SigToLogSig", "SigCombine",
           "SigJoin", "TransformPath"]
