"""Half-precision cast.  Reference: ``grace_dl/dist/compressor/fp16.py:6-22``."""
import torch

from ..core import Compressor


class FP16Compressor(Compressor):
    def compress(self, tensor, name):
        dtype = tensor.dtype
        if tensor.is_floating_point():
            tensor = tensor.to(torch.float16)
        return [tensor], dtype

    def decompress(self, tensors, ctx):
        (tensor,) = tensors
        if ctx is not None and ctx.is_floating_point:
            tensor = tensor.to(ctx)
        return tensor
