"""INCEPTIONN: per-element variable-width floating point truncation.

Reference: ``grace_dl/tensorflow/compressor/inceptionn.py:8-188`` (TensorFlow
only).  With ``e`` the biased exponent and ``eb = 127 + int(log10(bound/2))``,
``mid = eb + ceil((127-eb)/2)``:

* ``e >= 127``          -> kept as fp32            (class 3)
* ``mid <= e < 127``    -> 16-bit fixed point code (class 2)
* ``eb  <= e < mid``    -> 8-bit fixed point code  (class 1)
* ``e < eb``            -> dropped                 (class 0)

A fixed point code is the sign bit followed by the top bits of
``|x| * 2**(width-1)`` (|x| < 1), i.e. the significand shifted right by
``127 - e`` with its hidden one made explicit.  The class of every element is
packed four per byte.  Payload: ``(fp32[], 16-bit codes as byte pairs, uint8[],
uint8 classes)`` (byte tensors travel on every backend).
"""
import math

import torch

from ..core import Compressor


def pack2(classes: torch.Tensor) -> torch.Tensor:
    """Pack values in {0..3}, four per byte (element i -> bits 2*(i%4))."""
    pad = (-classes.numel()) % 4
    if pad:
        classes = torch.cat([classes, classes.new_zeros(pad)])
    c = classes.view(-1, 4).to(torch.int32)
    return (c[:, 0] | (c[:, 1] << 2) | (c[:, 2] << 4) | (c[:, 3] << 6)).to(torch.uint8)


def unpack2(packed: torch.Tensor, numel: int) -> torch.Tensor:
    p = packed.to(torch.int32)
    c = torch.stack([p & 3, (p >> 2) & 3, (p >> 4) & 3, (p >> 6) & 3], dim=1)
    return c.reshape(-1)[:numel]


class INCEPTIONNCompressor(Compressor):
    def __init__(self, error_bound):
        super().__init__(tensors_size_are_same=False)
        self.error_bound = error_bound
        self.exp_floor = 127 + int(math.log(error_bound / 2, 10))
        self.exp_mid = self.exp_floor + math.ceil((127 - self.exp_floor) / 2)

    @staticmethod
    def _fixed(x: torch.Tensor, width: int) -> torch.Tensor:
        """sign + (width-1) fractional bits of |x| < 1, truncated."""
        frac = torch.floor(x.abs().double() * (1 << (width - 1))).long()
        frac = frac.clamp(max=(1 << (width - 1)) - 1)
        return frac | ((x < 0).long() << (width - 1))

    @staticmethod
    def _unfixed(code: torch.Tensor, width: int) -> torch.Tensor:
        code = code.long() & ((1 << width) - 1)
        mag = (code & ((1 << (width - 1)) - 1)).double() / (1 << (width - 1))
        return torch.where((code >> (width - 1)) > 0, -mag, mag).float()

    def compress(self, tensor, name):
        flat = tensor.flatten().float()
        e = (flat.contiguous().view(torch.int32) >> 23) & 0xFF
        cls = torch.zeros_like(e)
        cls = torch.where((e >= self.exp_floor) & (e < self.exp_mid), torch.ones_like(e), cls)
        cls = torch.where((e >= self.exp_mid) & (e < 127), torch.full_like(e, 2), cls)
        cls = torch.where(e >= 127, torch.full_like(e, 3), cls)
        v32 = flat[cls == 3]
        v16 = self._fixed(flat[cls == 2], 16).to(torch.int16).view(torch.uint8)  # two bytes per code
        v8 = self._fixed(flat[cls == 1], 8).to(torch.uint8)
        return (v32, v16, v8, pack2(cls)), tensor.shape

    def decompress(self, tensors, ctx):
        v32, v16, v8, packed = tensors
        numel = ctx.numel()
        cls = unpack2(packed, numel)
        out = torch.zeros(numel, dtype=torch.float32, device=packed.device)
        out[cls == 3] = v32
        out[cls == 2] = self._unfixed(v16.contiguous().view(torch.int16), 16)
        out[cls == 1] = self._unfixed(v8, 8)
        return out.view(ctx)
