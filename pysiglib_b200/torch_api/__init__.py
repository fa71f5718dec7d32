"""Differentiable front-end (same names as the base package, no ``*_backprop``)."""
from ..sig_length import sig_length
from .torch_api import (Sig, SigCombine, SigJoin, TransformPath, sig, sig_combine, sig_join, signature,
                        transform_path)

__all__ = ["sig", "signature", "sig_combine", "sig_join", "transform_path", "sig_length", "Sig", "SigCombine",
           "SigJoin", "TransformPath"]
