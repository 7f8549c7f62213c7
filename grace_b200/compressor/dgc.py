"""Deep Gradient Compression selection.

Reference: ``grace_dl/dist/compressor/dgc.py:6-50``: estimate the top-``ratio``
magnitude threshold from a 1 % sample, then nudge it by x1.3 / x0.7 (at most ten
rounds, one host sync each) until the selected count lies in
``[0.7, 1.3] * ratio * N``.  ``mode='sampled'`` reproduces that procedure draw for
draw (same host-side uniform sample, hence the reference's selection for equal seeds); ``mode='exact'`` (default on CUDA) takes the exact k-th
magnitude from the radix-select kernel, which always lands inside the accepted
band and needs no host round trip.  ``ctx`` carries the selection mask that
``DgcMemory.update`` consumes.
"""
import torch

from ..core import Compressor
from ._common import scatter_dense, topk_count


class DgcCompressor(Compressor):
    def __init__(self, compress_ratio, mode=None):
        super().__init__(tensors_size_are_same=False)
        self.compress_ratio = compress_ratio
        self.mode = mode

    def _sampled_threshold(self, flat):
        numel = flat.numel()
        n_sample = max(1, int(numel * 0.01))
        # drawn exactly as the reference draws it (a float uniform on the host, truncated), so that equal seeds
        # give equal samples; the clamp covers the float rounding of `numel` itself for very large tensors
        sample_idx = torch.empty(n_sample).uniform_(0, numel).type(torch.long).clamp_(max=numel - 1).to(flat.device)
        k = max(1, int(numel * self.compress_ratio * 0.01))
        thr = torch.topk(flat[sample_idx].abs(), min(k, n_sample)).values.min()
        target = numel * self.compress_ratio
        mask = flat.abs() >= thr
        for _ in range(10):
            selected = int(mask.sum())
            if selected > 1.3 * target:
                thr = thr * 1.3
            elif selected < 0.7 * target:
                thr = thr * 0.7
            else:
                break
            mask = flat.abs() >= thr
        return mask

    def compress(self, tensor, name):
        flat = tensor.flatten()
        numel = flat.numel()
        mode = self.mode or ("exact" if flat.is_cuda else "sampled")
        if mode == "exact":
            k = topk_count(numel, self.compress_ratio)
            if flat.is_cuda:
                from ..ops import sparse as _sparse

                values, idx32 = _sparse.topk_select(flat, k)
                indices = idx32.long()
            else:
                _, indices = torch.topk(flat.abs(), k, sorted=False)
                values = flat[indices]
            mask = torch.zeros(numel, dtype=torch.bool, device=flat.device)
            mask[indices] = True
        else:
            mask = self._sampled_threshold(flat)
            (indices,) = torch.where(mask)
            values = flat[indices]
        return (values, indices), (tensor.shape, mask, numel)

    def decompress(self, tensors, ctx):
        values, indices = tensors
        shape, _, numel = ctx
        return scatter_dense(values, indices, numel).view(shape)
