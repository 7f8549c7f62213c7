"""Natural compression: stochastic rounding to a power of two, 8-bit code.

Two code tables exist in the reference (cupy: ``natural.py:8-40``; CUDA
extension: ``cnat_cuda/cnat_cuda.cu:68-134``).  This implements the CUDA
flavour: with ``x = m * 2**p`` and ``|m|`` in ``[0.5, 1)``, round to ``2**p``
with probability ``2|m| - 1`` else to ``2**(p-1)``; with ``B`` the biased
exponent of the result, the 7-bit code is 0 for ``B <= 17``, ``B - 17`` up to
127 (saturating), bit 7 is the sign.  ``deterministic=True`` rounds at
probability 0.5 (``cnat_compress_deterministic``).
"""
import torch

from ..core import Compressor
from ._common import StochasticMixin


def natural_encode(flat: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    bits = flat.contiguous().view(torch.int32)
    biased = (bits >> 23) & 0xFF
    mant = bits & 0x7FFFFF
    neg = bits < 0
    # |m| = (1 + mant/2^23)/2  ->  2|m| - 1 = mant / 2^23
    prob = mant.float() * (2.0 ** -23)
    up = u < prob
    b = biased + up.to(torch.int32)
    # denormals and zero have biased exponent 0 -> code 0
    code7 = torch.clamp(b - 17, min=0, max=127)
    code7 = torch.where(biased == 0, torch.zeros_like(code7), code7)
    return (code7 | (neg.to(torch.int32) << 7)).to(torch.uint8)


def natural_decode(code: torch.Tensor) -> torch.Tensor:
    c = code.to(torch.int32)
    code7 = c & 0x7F
    sign = (c >> 7) & 1
    bits = torch.where(code7 == 0, torch.zeros_like(c), (code7 + 17) << 23)
    # place the sign bit without overflowing int32 arithmetic
    out = bits.view(torch.float32)
    return torch.where(sign.bool(), -out, out)


class NaturalCompressor(StochasticMixin, Compressor):
    def __init__(self, deterministic=False):
        super().__init__()
        self.deterministic = deterministic

    def compress(self, tensor, name):
        flat = tensor.flatten().float()
        if flat.is_cuda:
            from ..ops import quant as _quant

            return [_quant.natural_compress(flat, name, self.deterministic)], tensor.shape
        if self.deterministic:
            # the reference keeps the larger power when 2|m|-1 > 0.5: u = 0 forces "up", u = 1 "down"
            bits = flat.contiguous().view(torch.int32)
            prob = (bits & 0x7FFFFF).float() * (2.0 ** -23)
            u = torch.where(prob > 0.5, torch.zeros_like(flat), torch.ones_like(flat))
        else:
            u = self._uniform(flat, name)
        return [natural_encode(flat, u)], tensor.shape

    def decompress(self, tensors, ctx):
        (code,) = tensors
        return natural_decode(code).view(ctx)


class NaturalCompressor_CUDA(NaturalCompressor):
    """Name kept for ``grace_from_params({'compressor': 'natural_cuda'})``."""
