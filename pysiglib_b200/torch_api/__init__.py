"""Differentiable front-end (same names as the base package, no ``*_backprop``)."""
from ..sig_length import sig_length
from .torch_api import Sig, sig, signature

__all__ = ["sig", "signature", "sig_length", "Sig"]
