"""Helpers shared by the compressors."""
from __future__ import annotations

from typing import Callable, Optional

import torch

UniformFn = Callable[[torch.Tensor, str], torch.Tensor]


def default_uniform(like: torch.Tensor, name: str) -> torch.Tensor:
    """fp32 U[0,1) samples shaped like ``like`` from torch's global generator."""
    return torch.rand(like.shape, dtype=torch.float32, device=like.device)


class StochasticMixin:
    """Gives a compressor a replaceable source of uniforms.

    Tests (and the deterministic-resume path) install a Philox stream that is
    bit-identical to the one the CUDA kernels consume; normal CPU use draws from
    torch's generator as the reference does.
    """

    uniform_fn: Optional[UniformFn] = None

    def _uniform(self, like: torch.Tensor, name: str) -> torch.Tensor:
        fn = self.uniform_fn or default_uniform
        return fn(like, name)


def topk_count(numel: int, ratio: float) -> int:
    """``k = max(1, int(N * ratio))`` as in ``grace_dl/dist/compressor/topk.py:34``."""
    return max(1, int(numel * ratio))


def scatter_dense(values: torch.Tensor, indices: torch.Tensor, numel: int) -> torch.Tensor:
    out = torch.zeros(numel, dtype=values.dtype, device=values.device)
    out.scatter_(0, indices.long(), values)
    return out
