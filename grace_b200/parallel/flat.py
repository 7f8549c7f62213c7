"""Flat parameter / gradient storage.

``FlatParams`` re-homes the parameters of a model into one flat fp32 buffer
and pre-allocates their ``.grad`` as views of a second flat buffer with the
same layout (every tensor starts on a 128-element boundary, memory order is
kept, so channels_last weights stay channels_last).  Backward then accumulates
straight into the flat gradient buffer, one fused exchange kernel handles a
whole bucket of named gradients, and one fused SGD kernel updates all
parameters.  The reference instead loops over ``model.named_parameters()`` in
Python and calls ``grc.step`` per tensor
(``examples/dist/CIFAR10-dawndist/core.py:203-206``).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch

from ..ops.exchange import ALIGN_ELEMS, FlatLayout


def _dense_view(flat: torch.Tensor, offset: int, like: torch.Tensor) -> torch.Tensor:
    n = like.numel()
    seg = flat[offset : offset + n]
    if like.is_contiguous() or n == 0:
        return seg.view(like.shape)
    # dense but permuted (e.g. channels_last): keep the strides
    return seg.as_strided(like.shape, like.stride())


class Bucket:
    """A contiguous range of the flat buffers with its own layout."""

    def __init__(self, index: int, start: int, end: int, names: List[str], numels: List[int], offsets: List[int],
                 shapes=None):
        self.index = index
        self.start, self.end = start, end
        self.layout = FlatLayout(names, numels, [o - start for o in offsets], end - start)
        self.layout.shapes = shapes
        self.pending = 0


class FlatParams:
    def __init__(self, named_parameters: Iterable[Tuple[str, torch.nn.Parameter]], bucket_bytes: Optional[int] = None,
                 grad_buffer=None):
        """``grad_buffer``: optional fp32 tensor, or a callable ``numel -> tensor or None``, that provides the
        storage of the flat gradient buffer (e.g. ``NvlsAllreduce.buffer`` so that gradients are reduced in place
        through the multicast mapping)."""
        named = [(n, p) for n, p in named_parameters if p.requires_grad]
        if not named:
            raise ValueError("no trainable parameters")
        dev = named[0][1].device
        for n, p in named:
            if p.dtype != torch.float32:
                raise TypeError("FlatParams keeps fp32 master parameters (use autocast for bf16 compute): %s is %s" % (n, p.dtype))
        self.names = [n for n, _ in named]
        self.params = [p for _, p in named]
        self.layout = FlatLayout.from_named([(n, p.numel()) for n, p in named])
        self.layout.shapes = [tuple(p.shape) for _, p in named]
        self.flat_p = torch.zeros(self.layout.total, dtype=torch.float32, device=dev)
        if callable(grad_buffer):
            grad_buffer = grad_buffer(self.layout.total)
        if grad_buffer is not None:
            if (grad_buffer.dtype != torch.float32 or grad_buffer.numel() < self.layout.total
                    or grad_buffer.device != dev or grad_buffer.data_ptr() % 16):
                raise ValueError("grad_buffer must be a 16-byte aligned fp32 tensor on %s with at least %d elements"
                                 % (dev, self.layout.total))
            self.flat_g = grad_buffer.reshape(-1)[: self.layout.total].zero_()
        else:
            self.flat_g = torch.zeros(self.layout.total, dtype=torch.float32, device=dev)
        with torch.no_grad():
            for p, off in zip(self.params, self.layout.offsets):
                view = _dense_view(self.flat_p, off, p.data)
                view.copy_(p.data)
                p.data = view
                p.grad = _dense_view(self.flat_g, off, p.data)
        self.buckets = self._make_buckets(bucket_bytes)
        self.bucket_of = {}
        for b in self.buckets:
            for n in b.layout.names:
                self.bucket_of[n] = b

    def _make_buckets(self, bucket_bytes: Optional[int]) -> List[Bucket]:
        lay = self.layout
        if not bucket_bytes:
            return [Bucket(0, 0, lay.total, list(lay.names), list(lay.numels), list(lay.offsets), list(lay.shapes))]
        limit = max(ALIGN_ELEMS, bucket_bytes // 4)
        buckets: List[Bucket] = []
        # gradients arrive roughly last parameter first: cut buckets from the end
        idx = len(lay.names)
        end = lay.total
        while idx > 0:
            j = idx
            while j > 0 and (end - lay.offsets[j - 1] <= limit or j == idx):
                j -= 1
            start = lay.offsets[j]
            buckets.append(Bucket(len(buckets), start, end, lay.names[j:idx], lay.numels[j:idx], lay.offsets[j:idx],
                                  lay.shapes[j:idx]))
            idx, end = j, start
        return buckets

    def grad_view(self, bucket: Bucket) -> torch.Tensor:
        return self.flat_g[bucket.start : bucket.end]

    def zero_grad(self):
        self.flat_g.zero_()

    def check_views(self) -> bool:
        """True while every ``.grad`` still aliases the flat gradient buffer."""
        base = self.flat_g.data_ptr()
        for p, off in zip(self.params, self.layout.offsets):
            if p.grad is None or p.grad.data_ptr() != base + 4 * off:
                return False
        return True

    def rebind_grads(self):
        for p, off in zip(self.params, self.layout.offsets):
            p.grad = _dense_view(self.flat_g, off, p.data)
