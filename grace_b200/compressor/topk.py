"""Top-k sparsification by magnitude.

Reference: ``grace_dl/dist/compressor/topk.py:32-69`` (``kernel='torch'``),
``radixtopk_cuda/rdxtopk_cuda.cu`` (``kernel='rdxtopk_cuda'``) and the cupy
partition variant.  Here ``kernel`` is accepted for API compatibility; on a CUDA
tensor every value of it runs the in-tree radix-select kernel
(``csrc/sparse_exchange.cu``), on CPU ``torch.topk``.
Payload: ``[values fp32 k, indices int32 k]``; ``k = max(1, int(N*ratio))``.
"""
import torch

from ..core import Compressor
from ._common import scatter_dense, topk_count


def sparsify(tensor: torch.Tensor, compress_ratio: float):
    flat = tensor.flatten()
    k = topk_count(flat.numel(), compress_ratio)
    if flat.is_cuda:
        from ..ops import sparse as _sparse

        return _sparse.topk_select(flat, k)
    _, idx = torch.topk(flat.abs(), k, sorted=False)
    return flat[idx], idx.to(torch.int32)


def desparsify(values, indices, numel):
    return scatter_dense(values, indices, numel)


class TopKCompressor(Compressor):
    def __init__(self, compress_ratio, kernel="torch"):
        super().__init__()
        self.compress_ratio = compress_ratio
        self.kernel = kernel

    def compress(self, tensor, name):
        values, indices = sparsify(tensor, self.compress_ratio)
        return [values, indices], (tensor.numel(), tensor.shape)

    def decompress(self, tensors, ctx):
        values, indices = tensors
        numel, shape = ctx
        return desparsify(values, indices, numel).view(shape)
