#!/usr/bin/env python
"""The reference ships two eyeball demos for its extensions (``radixtopk_cuda/example.py:10-28`` prints
``rdxtopk.topk`` next to ``torch.topk`` for 500 000 random floats; ``qsgd_cuda/example.py:9-16`` prints a QSGD
round trip of 200 000 floats).  This script runs the same calls through the same module names and CHECKS the
results instead of printing them for inspection.  Uses the GPU kernels when a GPU is present, torch ops otherwise.

    python examples/native_ops_demo.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import cnat_cuda
import qsgd_cuda
import rdxtopk


def main():
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    x = torch.rand(500_000, device=dev)
    k = 5000
    vals, idx = rdxtopk.topk(x, torch.arange(x.numel(), device=dev).int(), k)
    ref_vals, _ = torch.topk(x, k)
    same = torch.equal(vals.sort().values, ref_vals.sort().values) and torch.equal(x[idx.long()], vals)
    print("rdxtopk.topk: k=%d  min %.6f  max %.6f  equals torch.topk: %s" % (k, vals.min(), vals.max(), same))

    y = torch.rand(200_000, device=dev) - 0.5
    codes, norms = qsgd_cuda.compress(y, 127, 128)
    back = qsgd_cuda.decompress(codes, norms, 127, 128)
    step = norms.float().repeat_interleave(128)[: y.numel()] / 127
    ok = bool(((back - y).abs() <= step + 1e-6).all())
    print("qsgd_cuda: %d B -> %d B, max error %.3e (one level = %.3e): within one level: %s"
          % (y.numel() * 4, codes.numel() + norms.numel() * 4, (back - y).abs().max(), step.max(), ok))

    z = torch.randn(200_000, device=dev) * 1e-3
    dec = cnat_cuda.decompress(cnat_cuda.compress(z))
    ratio = dec.abs() / z.abs()
    ok2 = bool(((ratio >= 0.5) & (ratio <= 2.0)).all())
    print("cnat_cuda: %d B -> %d B, mean ratio %.4f (unbiased: ~1), neighbouring powers of two: %s"
          % (z.numel() * 4, z.numel(), float((dec / z).mean()), ok2))
    if not (same and ok and ok2):
        raise SystemExit(1)


if __name__ == "__main__":
    main()
