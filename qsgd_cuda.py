"""``qsgd_cuda.compress(input, level, bucket) -> (int8 codes, float64 norms)`` and
``qsgd_cuda.decompress(codes, norms, level, bucket) -> float32`` with the signatures of the reference's QSGD
extension (``grace_dl/dist/compressor/qsgd_cuda/qsgd.cpp:1-24``, kernels ``qsgd_cuda.cu:320-408``): per-bucket L2
norm, stochastic rounding to ``level`` levels, decode ``norm / level * code``.  CUDA tensors with bucket 128 and
fewer than 128 levels run the in-tree sm_100a encoder; other inputs run the torch implementation.  A bucket
whose norm is zero encodes to zeros (the reference produces NaN there).
"""
import torch

from grace_b200.compressor.qsgd import QSGDCompressor


def compress(input: torch.Tensor, level: int, bucket: int = 128):
    flat = input.reshape(-1)
    comp = QSGDCompressor(int(level), int(bucket))
    if flat.is_cuda and (int(bucket) != 128 or int(level) >= 128):
        (codes, norms), _ = comp.compress(flat.cpu(), "qsgd_cuda")     # shapes the kernel does not cover
        codes, norms = codes.to(flat.device), norms.to(flat.device)
    else:
        (codes, norms), _ = comp.compress(flat, "qsgd_cuda")
    return codes, norms.double()


def decompress(codes: torch.Tensor, norms: torch.Tensor, level: int, bucket: int = 128) -> torch.Tensor:
    comp = QSGDCompressor(int(level), int(bucket))
    return comp.decompress((codes, norms.float()), torch.Size([codes.numel()]))
