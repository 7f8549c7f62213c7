"""Random-k sparsification with rank-agreed indices.

Reference: ``grace_dl/dist/compressor/randomk.py:6-41``.  All ranks derive the
same indices from ``sum(utf8(name)) + global_step`` so only values travel and
the payload is all-reduce friendly.  The reference re-seeds torch's *global*
generator on every call; here a private ``torch.Generator`` is seeded instead,
which gives the same index stream on CPU without the side effect.  Indices are
drawn with replacement (dist flavour); ``with_replacement=False`` gives the
permutation-prefix behaviour of ``grace_dl/torch/compressor/randomk.py:10``.
"""
import torch

from ..core import Compressor
from ._common import topk_count


def name_seed(name: str, step: int) -> int:
    return sum(bytes(name, encoding="utf8"), step)


class RandomKCompressor(Compressor):
    _state_fields = ("global_step",)

    def __init__(self, compress_ratio, with_replacement=True):
        super().__init__()
        self.global_step = 0
        self.compress_ratio = compress_ratio
        self.with_replacement = with_replacement

    def indices_for(self, name, numel, device):
        gen = torch.Generator(device="cpu")
        gen.manual_seed(name_seed(name, self.global_step))
        k = topk_count(numel, self.compress_ratio)
        if self.with_replacement:
            idx = torch.randint(numel, [k], generator=gen)
        else:
            idx = torch.randperm(numel, generator=gen)[:k]
        return idx.to(device)

    def compress(self, tensor, name):
        flat = tensor.flatten()
        indices = self.indices_for(name, flat.numel(), flat.device)
        self.global_step += 1
        return [flat[indices]], (indices, flat.numel(), tensor.shape)

    def decompress(self, tensors, ctx):
        indices, numel, shape = ctx
        (values,) = tensors
        out = torch.zeros(numel, dtype=values.dtype, device=values.device)
        out.scatter_(0, indices, values)
        return out.view(shape)
