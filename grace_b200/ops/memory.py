"""Stand-alone error-feedback kernels for CUDA tensors (``csrc/memory.cu``).

Used by the memory classes when ``compensate`` / ``update`` are called one by one (the library communicators, user
code following the reference's ``Communicator.step``): one streaming kernel per call instead of a chain of eager ops
(``grace_dl/dist/memory/residual.py:10-20``, ``memory/dgc.py:15-39``).  Gradients may be fp32, bf16 or fp16; state
tensors are fp32.  Every function returns None when the tensor is not eligible (CPU, other dtype, not dense), and
the caller then uses its torch-op path.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from .exchange import GRAD_DTYPE


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def eligible(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype in GRAD_DTYPE and t.is_contiguous()
            and t.data_ptr() % (16 if t.dtype == torch.float32 else 8) == 0 and 0 < t.numel() < 2 ** 40)


def _state_ok(*ts) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.data_ptr() % 16 == 0)
               for t in ts)


def residual_compensate(g: torch.Tensor, residual: Optional[torch.Tensor], beta: float, gamma: float):
    """``beta * residual + gamma * g`` as a new fp32 tensor shaped like ``g`` (``residual`` None: ``gamma * g``)."""
    if not eligible(g) or not _state_ok(residual):
        return None
    out = torch.empty(g.shape, dtype=torch.float32, device=g.device)
    native().residual_compensate(g.data_ptr(), GRAD_DTYPE[g.dtype], residual.data_ptr() if residual is not None else 0,
                                 out.data_ptr(), g.numel(), float(beta), float(gamma), _stream())
    return out


def residual_update(acc: torch.Tensor, decompressed: torch.Tensor):
    """``acc - decompressed`` as a new fp32 tensor."""
    if not (eligible(acc) and acc.dtype == torch.float32 and _state_ok(decompressed)
            and decompressed.numel() == acc.numel()):
        return None
    out = torch.empty_like(acc)
    native().residual_update(acc.data_ptr(), decompressed.data_ptr(), out.data_ptr(), acc.numel(), _stream())
    return out


def sparse_residual(acc: torch.Tensor, indices: torch.Tensor):
    """Copy of ``acc`` with the transmitted positions zeroed: the residual of a sparse codec without a dense decompress."""
    if not (eligible(acc) and acc.dtype == torch.float32 and indices.is_cuda and indices.is_contiguous()
            and indices.dtype in (torch.int32, torch.int64)):
        return None
    out = acc.clone()
    native().zero_at(out.data_ptr(), 0, indices.data_ptr(), int(indices.dtype == torch.int64), indices.numel(),
                     out.numel(), _stream())
    return out


def dgc_compensate(g: torch.Tensor, u: torch.Tensor, v: torch.Tensor, momentum: float, bound: float, first: bool) -> bool:
    """In place: ``u = momentum * u + clamp(g, -bound, bound)``, ``v += u`` (``first``: u and v start from zero)."""
    if not eligible(g) or not _state_ok(u, v) or u.numel() != g.numel() or v.numel() != g.numel():
        return False
    native().dgc_compensate(g.data_ptr(), GRAD_DTYPE[g.dtype], u.data_ptr(), v.data_ptr(), g.numel(), float(momentum),
                            float(bound), int(first), _stream())
    return True


def dgc_mask(u: torch.Tensor, v: torch.Tensor, mask: torch.Tensor) -> bool:
    """In place: zero ``u`` and ``v`` where ``mask`` (bool / uint8, one per element) is set."""
    if not _state_ok(u, v) or not mask.is_cuda or mask.numel() != u.numel() or mask.dtype not in (torch.bool, torch.uint8):
        return False
    m = mask.contiguous().view(torch.uint8)
    native().dgc_mask(u.data_ptr(), v.data_ptr(), m.data_ptr(), u.numel(), _stream())
    return True


_scratch = {}


def sum_squares(g: torch.Tensor):
    """``sum(g^2)`` as a 0-d fp64 tensor on the device (fixed-order reduction: the same bits on every run)."""
    if not eligible(g):
        return None
    C = native()
    key = (g.device, torch.cuda.current_stream().cuda_stream)
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = torch.zeros(C.sum_squares_scratch_doubles(), dtype=torch.float64, device=g.device)
    C.sum_squares(g.data_ptr(), GRAD_DTYPE[g.dtype], g.numel(), buf.data_ptr(), _stream())
    return buf[0].clone()
