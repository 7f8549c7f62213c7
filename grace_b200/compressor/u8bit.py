"""8-bit non-uniform quantisation (Dettmers, "8-Bit Approximations for
Parallelism in Deep Learning").

Reference: ``grace_dl/tensorflow/compressor/u8bit.py:6-110`` (TensorFlow only
there).  ``s = max|x|``; ``bin`` = index of the interval of the 128-entry table
that holds ``|x|/s``; code ``= int8(bin) * sign(x)``; decode = lower edge of the
bin times ``s`` times the sign, and bin 0 decodes to 0 because ``sign(0) = 0``.
Values below the first edge go to bin 0 and values above the last edge to bin
126 (the reference yields NaN bins there).
"""
import torch

from ..core import Compressor

# Bin edges of the 8-bit dynamic-tree data type; numeric data of the algorithm.
_HEAD = [1.5000001e-06, 2.7500000e-06, 7.2499997e-06, 1.8750001e-05, 3.6250000e-05, 5.8749996e-05, 8.6249995e-05]


def _build_edges():
    """The table is piecewise linear: runs of equal spacing that double in
    step from decade to decade.  It is generated here and rounded to fp32; the
    generated values agree with the published 128-entry table to within one
    fp32 ulp (the published list carries accumulated rounding noise)
    (checked by the unit tests against literal spot values)."""
    edges = list(_HEAD)
    runs = [
        (1.4375e-04, 8.75e-05, 4),       # 1.4375e-4 .. 4.0625e-4
        (5.1875e-04, 1.375e-04, 4),      # .. 9.3125e-4
        (1.21875e-03, 4.375e-04, 8),     # .. 4.28125e-3
        (4.84375e-03, 6.875e-04, 8),     # .. 9.65625e-3
        (1.109375e-02, 2.1875e-03, 16),  # .. 4.390625e-2
        (4.671875e-02, 3.4375e-03, 16),  # .. 9.828125e-2
        (1.0546875e-01, 1.09375e-02, 32),  # .. 4.4453125e-1
        (4.5859375e-01, 1.71875e-02, 32),  # .. 9.9140625e-1
    ]
    for start, step, count in runs:
        edges.extend(start + i * step for i in range(count))
    edges.append(9.9570298e-01)
    assert len(edges) == 128, len(edges)
    return edges


DICT128 = torch.tensor(_build_edges(), dtype=torch.float32)


class U8bitCompressor(Compressor):
    def __init__(self):
        super().__init__()
        self._edges = {}

    def _table(self, device):
        key = str(device)
        if key not in self._edges:
            self._edges[key] = DICT128.to(device)
        return self._edges[key]

    def compress(self, tensor, name):
        flat = tensor.flatten().float()
        edges = self._table(flat.device)
        scale = flat.abs().max()
        safe = torch.where(scale > 0, scale, torch.ones_like(scale))
        y = flat.abs() / safe
        # interval index: edges[i] <= y < edges[i+1]
        bins = torch.bucketize(y, edges, right=True) - 1
        bins = bins.clamp(0, 126)
        code = (bins * flat.sign().to(bins.dtype)).to(torch.int8)
        return (code, scale.reshape(1)), tensor.shape

    def decompress(self, tensors, ctx):
        code, scale = tensors
        edges = self._table(code.device)
        c = code.to(torch.int64)
        return (edges[c.abs()] * scale * c.sign().float()).view(ctx)
