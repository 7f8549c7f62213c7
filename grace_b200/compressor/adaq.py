"""AdaComp-style two-sided sparse quantisation ("adaq").

Reference: ``grace_dl/tensorflow/compressor/adaq.py:6-93`` (TensorFlow only).
Positive and negative parts are treated separately: each keeps roughly
``ratio`` of its elements (largest magnitude) and transmits only their indices
plus one mean value per side.  The reference estimates each threshold from a
1 % sample with a correction loop; here the exact k-th magnitude is used,
which always satisfies the reference's acceptance band ``[0.8, 1.25]*k``.
Payload: one int32 tensor ``[mean+ bits, mean- bits, n+, idx+..., idx-...]``.
"""
import math

import torch

from ..core import Compressor


class AdaqCompressor(Compressor):
    def __init__(self, compress_ratio):
        super().__init__(tensors_size_are_same=False)
        self.compress_ratio = compress_ratio

    def _side(self, flat, side_mask):
        count = int(side_mask.sum())
        if count == 0:
            return flat.new_zeros((), dtype=torch.float32), torch.empty(0, dtype=torch.int32, device=flat.device)
        k = max(1, int(math.ceil(count * self.compress_ratio)))
        mag = torch.where(side_mask, flat.abs(), flat.new_zeros(()))
        vals, idx = torch.topk(mag, min(k, count), sorted=False)
        idx = idx.sort().values
        return flat[idx].mean(), idx.to(torch.int32)

    def compress(self, tensor, name):
        flat = tensor.flatten().float()
        mean_p, idx_p = self._side(flat, flat > 0)
        mean_n, idx_n = self._side(flat, flat < 0)
        head = torch.stack([mean_p, mean_n]).view(torch.int32)
        n_p = torch.tensor([idx_p.numel()], dtype=torch.int32, device=flat.device)
        return [torch.cat([head, n_p, idx_p, idx_n])], (tensor.shape, flat.numel())

    def decompress(self, tensors, ctx):
        (packed,) = tensors
        shape, numel = ctx
        means = packed[:2].view(torch.float32)
        n_p = int(packed[2])
        idx_p = packed[3 : 3 + n_p].long()
        idx_n = packed[3 + n_p :].long()
        out = torch.zeros(numel, dtype=torch.float32, device=packed.device)
        out[idx_p] = means[0]
        out[idx_n] = means[1]
        return out.view(shape)
