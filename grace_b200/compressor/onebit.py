"""1-bit SGD: sign mask plus the means of the two halves.

Reference: ``grace_dl/dist/compressor/onebit.py:6-31`` with the decode of
``grace_dl/torch/compressor/onebit.py:27-32`` (the dist copy applies ``~`` to a
uint8 mask, which is a bitwise not and produces garbage).
"""
import torch

from ..core import Compressor


class OneBitCompressor(Compressor):
    def compress(self, tensor, name):
        flat = tensor.flatten()
        neg = flat < 0
        n_neg = neg.sum()
        n_pos = flat.numel() - n_neg
        zero = flat.new_zeros(())
        sum_neg = torch.where(neg, flat, zero).sum()
        sum_pos = torch.where(neg, zero, flat).sum()
        mean0 = torch.where(n_neg > 0, sum_neg / n_neg.clamp(min=1), sum_neg)
        mean1 = torch.where(n_pos > 0, sum_pos / n_pos.clamp(min=1), sum_pos)
        return (neg.to(torch.uint8), mean0, mean1), tensor.shape

    def decompress(self, tensors, ctx):
        mask0, mean0, mean1 = tensors
        return torch.where(mask0.bool(), mean0, mean1).view(ctx)
