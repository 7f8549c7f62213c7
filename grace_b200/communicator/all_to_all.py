"""Compressed reduce-scatter followed by a compressed all-gather.

Reference: ``grace_dl/dist/communicator/all_to_all.py:13-124``.  The element
codes are cut into W chunks; chunk j goes to rank j, which decodes the W
chunks it received, sums them, encodes the sum again (a second lossy step) and
all-gathers the result.  Supported codecs: QSGD (codes + per-bucket norms),
TernGrad (codes + one scale) and natural compression (codes only).  Padding is
zero-filled (the reference pads with uninitialised memory).
"""
import math

import torch
from torch import distributed as dist

from ..core import Communicator
from ..compressor.natural import NaturalCompressor
from ..compressor.qsgd import QSGDCompressor
from ..compressor.terngrad import TernGradCompressor
from . import _dist


def _pad_to(t: torch.Tensor, numel: int) -> torch.Tensor:
    if t.numel() == numel:
        return t
    out = t.new_zeros(numel)
    out[: t.numel()] = t
    return out


class AllToAll(Communicator):
    def _exchange(self, data: torch.Tensor):
        chunks = list(data.chunk(self.world_size))
        out = [torch.empty_like(c) for c in chunks]
        _dist.all_to_all(out, chunks)
        return out

    def _gather_decode(self, payload, ctx):
        columns = []
        for t in payload:
            out = [torch.empty_like(t) for _ in range(self.world_size)]
            dist.all_gather(out, t.contiguous())
            columns.append(out)
        return torch.cat([self.compressor.decompress(list(p), ctx).flatten() for p in zip(*columns)])

    def send_receive(self, tensors, name, ctx):
        comp = self.compressor
        W = self.world_size
        if not (_dist.active() and W > 1):
            out = comp.decompress(tensors, ctx)
            return out
        if isinstance(comp, QSGDCompressor):
            codes, norms = tensors
            numel = codes.numel()
            B = comp.bucket_size
            padded = math.ceil(numel / (W * B)) * W * B
            code_chunks = self._exchange(_pad_to(codes, padded))
            norm_chunks = self._exchange(_pad_to(norms, padded // B))
            parts = [comp.decompress((c, n), c.shape) for c, n in zip(code_chunks, norm_chunks)]
        elif isinstance(comp, TernGradCompressor):
            codes, scale = tensors
            numel = codes.numel()
            padded = math.ceil(numel / W) * W
            code_chunks = self._exchange(_pad_to(codes, padded))
            scales = [torch.empty_like(scale) for _ in range(W)]
            dist.all_gather(scales, scale)
            parts = [comp.decompress((c, s), c.shape) for c, s in zip(code_chunks, scales)]
        elif isinstance(comp, NaturalCompressor):
            (codes,) = tensors
            numel = codes.numel()
            padded = math.ceil(numel / W) * W
            parts = [comp.decompress([c], c.shape) for c in self._exchange(_pad_to(codes, padded))]
        else:
            raise NotImplementedError("AllToAll supports QSGD, TernGrad and natural compression, got %r" % comp)
        reduced = comp.aggregate(parts)
        payload2, ctx2 = comp.compress(reduced, name)
        full = self._gather_decode(payload2, ctx2)
        shape = ctx if isinstance(ctx, torch.Size) else ctx
        out = full[:numel].view(shape)
        return out / W if comp.average else out
