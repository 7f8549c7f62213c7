"""QSGD: bucketed stochastic uniform quantisation.

Reference: ``grace_dl/dist/compressor/qsgd.py:5-51`` (torch ops) and
``qsgd_cuda/qsgd_cuda.cu`` (``QSGDCompressor_CUDA``).  Per bucket ``b`` of
``bucket_size`` consecutive elements: ``l = q*|x|/||b||``,
``level = floor(l) + [u < frac(l)]``, code ``= sign(x)*level`` stored as int8
when ``q < 128`` else fp16; decode ``||b||/q * code``.  A zero-norm bucket
encodes to zeros (the reference divides 0/0 there).
"""
import torch

from ..core import Compressor
from ._common import StochasticMixin


def _bucketed(flat: torch.Tensor, bucket: int) -> torch.Tensor:
    pad = (-flat.numel()) % bucket
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    return flat.view(-1, bucket)


class QSGDCompressor(StochasticMixin, Compressor):
    def __init__(self, quantum_num, bucket_size=128):
        super().__init__()
        self.quantum_num = quantum_num
        self.bucket_size = bucket_size

    def compress(self, tensor, name):
        shape = tensor.shape
        flat = tensor.flatten().float()
        numel = flat.numel()
        if flat.is_cuda:
            from ..ops import quant as _quant

            codes, norms = _quant.qsgd_compress(flat, self.quantum_num, self.bucket_size, name)
            return (codes, norms), shape
        buckets = _bucketed(flat, self.bucket_size)
        bucket_norm = buckets.pow(2).sum(dim=1).sqrt()
        norm = bucket_norm.repeat_interleave(self.bucket_size)[:numel]
        safe = torch.where(norm > 0, norm, torch.ones_like(norm))
        level_float = self.quantum_num / safe * flat.abs()
        lower = level_float.floor()
        u = self._uniform(flat, name)
        level = lower + (u < (level_float - lower)).float()
        level = torch.where(norm > 0, level, torch.zeros_like(level))
        code = (level * flat.sign()).to(torch.int16)
        code = code.to(torch.int8 if self.quantum_num < 128 else torch.half)
        return (code, bucket_norm), shape

    def decompress(self, tensors, ctx):
        code, bucket_norm = tensors
        numel = ctx.numel() if isinstance(ctx, torch.Size) else int(torch.Size(ctx).numel())
        norm = bucket_norm.float().repeat_interleave(self.bucket_size)[:numel]
        return (norm / self.quantum_num * code.float()).view(ctx)


class QSGDCompressor_CUDA(QSGDCompressor):
    """Name kept for ``grace_from_params({'compressor': 'qsgd_cuda'})``.

    The reference routes this class to a separate extension; here both names
    run the same in-tree kernel on CUDA tensors.
    """
