"""Differentiable front-end (same names as the base package, no ``*_backprop``)."""
from ..sig_length import sig_length
from .torch_api import (Sig, SigCombine, SigJoin, SigToLogSig, TransformPath, log_sig, sig, sig_combine, sig_join,
                        sig_to_log_sig, signature, transform_path)

__all__ = ["sig", "signature", "sig_combine", "sig_join", "transform_path", "log_sig", "sig_to_log_sig", "sig_length", "Sig", "SigToLogSig", "SigCombine",
           "SigJoin", "TransformPath"]
