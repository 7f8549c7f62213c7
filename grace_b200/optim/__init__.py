"""Optimizers backed by hand-written kernels."""
from .fused_sgd import FusedSGD

__all__ = ["FusedSGD"]
