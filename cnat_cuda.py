"""``cnat_cuda.compress / compress_deterministic / decompress`` with the signatures of the reference's natural
compression extension (``grace_dl/dist/compressor/cnat_cuda/cnat.cpp:1-29``, kernels ``cnat_cuda.cu:68-134``):
fp32 -> one byte (sign + 7-bit exponent code, exponent rounded up with probability mantissa / 2^23, or to the
nearest power of two in the deterministic variant) and back.  CUDA tensors run the in-tree sm_100a encoder
(Philox in registers); CPU tensors run the same code table in torch ops.
"""
import torch

from grace_b200.compressor.natural import NaturalCompressor, natural_decode

_stochastic = NaturalCompressor(deterministic=False)
_deterministic = NaturalCompressor(deterministic=True)


def compress(tensor: torch.Tensor) -> torch.Tensor:
    (code,), _ = _stochastic.compress(tensor.reshape(-1), "cnat_cuda")
    return code


def compress_deterministic(tensor: torch.Tensor) -> torch.Tensor:
    (code,), _ = _deterministic.compress(tensor.reshape(-1), "cnat_cuda")
    return code


def decompress(code: torch.Tensor) -> torch.Tensor:
    return natural_decode(code)
