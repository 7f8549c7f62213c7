"""Error-feedback signSGD: sign plus the mean magnitude.

Reference: ``grace_dl/dist/compressor/efsignsgd.py:6-33``; aggregate is
``sum_r mean_r * sign_r / lr`` and is not averaged.
"""
import torch

from ..core import Compressor


class EFSignSGDCompressor(Compressor):
    def __init__(self, lr):
        super().__init__(average=False)
        self.learning_rate = lr

    def compress(self, tensor, name):
        flat = tensor.flatten()
        return (flat.abs().mean(), (flat >= 0).to(torch.uint8)), tensor.shape

    def decompress(self, tensors, ctx):
        mean, bits = tensors
        return (mean * (bits.float() * 2 - 1)).view(ctx)

    def aggregate(self, tensors):
        total = tensors[0].clone()
        for t in tensors[1:]:
            total += t
        return total / self.learning_rate
