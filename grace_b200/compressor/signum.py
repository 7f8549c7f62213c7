"""Signum: sign of a per-tensor momentum, majority vote.

Reference: ``grace_dl/dist/compressor/signum.py:6-37``:
``m = (1-beta)*g + beta*m`` (first step ``m = g``), payload ``m >= 0``.
"""
import torch

from ..core import Compressor
from .signsgd import majority_vote


class SignumCompressor(Compressor):
    _state_fields = ("momentums",)

    def __init__(self, momentum):
        super().__init__(average=False)
        self.momentum = momentum
        self.momentums = {}

    def compress(self, tensor, name):
        flat = tensor.flatten()
        if name in self.momentums:
            flat = (1.0 - self.momentum) * flat + self.momentum * self.momentums[name]
        self.momentums[name] = flat
        return [(flat >= 0).to(torch.uint8)], tensor.shape

    def decompress(self, tensors, ctx):
        (bits,) = tensors
        return (bits.float() * 2 - 1).view(ctx)

    def aggregate(self, tensors):
        return majority_vote(tensors)
