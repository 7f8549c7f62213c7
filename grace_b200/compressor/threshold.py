"""Magnitude threshold sparsification (variable-size payload).

Reference: ``grace_dl/dist/compressor/threshold.py:6-27``: keep every element
with ``|x| >= min(threshold, max(x))``.  The Horovod flavour of the reference
(``grace_dl/torch/compressor/threshold.py:17``) keeps ``|x| > threshold`` without the
cap; ``strict=True`` selects that rule (the ``grace_dl.torch`` import path does).
"""
import torch

from ..core import Compressor
from ._common import scatter_dense


class ThresholdCompressor(Compressor):
    def __init__(self, threshold, strict=False):
        super().__init__(tensors_size_are_same=False)
        self.threshold = threshold
        self.strict = strict

    def compress(self, tensor, name):
        flat = tensor.flatten()
        if self.strict:
            (indices,) = torch.where(flat.abs() > self.threshold)
        else:
            thr = torch.clamp(flat.max(), max=self.threshold)
            (indices,) = torch.where(flat.abs() >= thr)
        return [flat[indices], indices.to(torch.int32)], tensor.shape

    def decompress(self, tensors, ctx):
        values, indices = tensors
        return scatter_dense(values, indices, ctx.numel()).view(ctx)
