"""Identity codec.  Reference: ``grace_dl/dist/compressor/none.py:4-12``."""
from ..core import Compressor


class NoneCompressor(Compressor):
    def compress(self, tensor, name):
        return [tensor], None

    def decompress(self, tensors, ctx):
        (tensor,) = tensors
        return tensor
