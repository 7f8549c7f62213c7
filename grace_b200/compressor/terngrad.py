"""TernGrad: stochastic ternarisation with 2.5-sigma clipping.

Reference: ``grace_dl/dist/compressor/terngrad.py:5-30``.
Payload ``(int8 N in {-1,0,1}, fp32 [1])``; decode ``t * s``.
"""
import torch

from ..core import Compressor
from ._common import StochasticMixin


class TernGradCompressor(StochasticMixin, Compressor):
    def compress(self, tensor, name):
        shape = tensor.shape
        flat = tensor.flatten().float()
        if flat.is_cuda:
            from ..ops import quant as _quant

            codes, scale = _quant.terngrad_compress(flat, name)
            return (codes, scale), shape
        std = (flat - flat.mean()).pow(2).mean().sqrt()
        c = 2.5 * std
        clipped = torch.maximum(torch.minimum(flat, c), -c)
        mag = clipped.abs()
        scalar = mag.max()
        u = self._uniform(flat, name) * scalar
        tern = torch.where(u >= mag, torch.zeros_like(clipped), clipped.sign())
        return (tern.to(torch.int8), scalar.reshape(1)), shape

    def decompress(self, tensors, ctx):
        tern, scalar = tensors
        return (tern.float() * scalar).view(ctx)
