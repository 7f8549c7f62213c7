"""Magnitude threshold sparsification (variable-size payload).

Reference: ``grace_dl/dist/compressor/threshold.py:6-27``: keep every element
with ``|x| >= min(threshold, max(x))``.
"""
import torch

from ..core import Compressor
from ._common import scatter_dense


class ThresholdCompressor(Compressor):
    def __init__(self, threshold):
        super().__init__(tensors_size_are_same=False)
        self.threshold = threshold

    def compress(self, tensor, name):
        flat = tensor.flatten()
        thr = torch.clamp(flat.max(), max=self.threshold)
        (indices,) = torch.where(flat.abs() >= thr)
        return [flat[indices], indices.to(torch.int32)], tensor.shape

    def decompress(self, tensors, ctx):
        values, indices = tensors
        return scatter_dense(values, indices, ctx.numel()).view(ctx)
