"""SketchML-style quantile bucketing.

Reference: ``grace_dl/tensorflow/compressor/sketch.py:6-39`` (TensorFlow only):
split the value range at ``quantiles`` equally populated cut points, send each
element's bin id (uint8, or int16 when more than 255 bins) and the mean of each
bin; decode by table lookup.
"""
import torch

from ..core import Compressor


class SketchCompressor(Compressor):
    def __init__(self, quantiles):
        super().__init__()
        self.quantiles = quantiles

    def compress(self, tensor, name):
        flat = tensor.flatten().float()
        q = self.quantiles
        probs = torch.linspace(0, 1, q + 1, device=flat.device)
        # torch.quantile limits input size; a sorted-lookup is equivalent
        srt = flat.sort().values
        pos = probs * (flat.numel() - 1)
        lo = pos.floor().long()
        hi = pos.ceil().long()
        frac = pos - lo
        edges = srt[lo] * (1 - frac) + srt[hi] * frac
        bins = (torch.bucketize(flat, edges[1:-1], right=True)).clamp(0, q - 1)
        sums = torch.zeros(q, device=flat.device).scatter_add_(0, bins, flat)
        cnts = torch.zeros(q, device=flat.device).scatter_add_(0, bins, torch.ones_like(flat))
        means = sums / cnts.clamp(min=1)
        code = bins.to(torch.uint8 if q < 256 else torch.int16)
        return (code, means), tensor.shape

    def decompress(self, tensors, ctx):
        code, means = tensors
        return means[code.long()].view(ctx)
