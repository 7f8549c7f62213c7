"""signSGD with majority vote.

Reference: ``grace_dl/dist/compressor/signsgd.py:6-30``.  The stand-alone
payload is one uint8 per element as in the reference; the fused exchange packs
32 signs per word.
"""
import torch

from ..core import Compressor


def majority_vote(tensors):
    total = tensors[0].clone()
    for t in tensors[1:]:
        total += t
    return torch.where(total >= 0, torch.ones_like(total), -torch.ones_like(total))


class SignSGDCompressor(Compressor):
    def __init__(self):
        super().__init__(average=False)

    def compress(self, tensor, name):
        flat = tensor.flatten()
        return [(flat >= 0).to(torch.uint8)], tensor.shape

    def decompress(self, tensors, ctx):
        (bits,) = tensors
        return (bits.float() * 2 - 1).view(ctx)

    def aggregate(self, tensors):
        return majority_vote(tensors)
