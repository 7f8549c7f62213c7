"""PowerSGD: rank-r approximation by one step of subspace iteration.

Reference: ``grace_dl/dist/compressor/powersgd.py:7-65``.  1-D tensors pass
through.  Otherwise ``M = g.view(shape[0], -1)``, ``P = M Q`` -> mean over
ranks -> Gram-Schmidt -> ``Q = M^T P`` -> mean over ranks; the payload is empty
and ``(P, Q, shape)`` is the context, so the collectives happen inside
``compress``.  ``all_reduce_fn`` is injectable (the fused path replaces the two
collectives and the three GEMMs by one kernel launch; tests inject a fake).

Differences from the reference, all on purpose: ``rank`` and ``world_size``
given to the factory actually reach this class; ``q_memory`` warm start is real
when ``use_memory=True``.
"""
import torch
from torch import distributed as dist

from ..core import Compressor


def orthogonalize(matrix: torch.Tensor) -> None:
    """In-place modified Gram-Schmidt over columns, no epsilon
    (``powersgd.py:7-18`` of the reference)."""
    cols = matrix.shape[1]
    for i in range(cols):
        col = matrix[:, i : i + 1]
        col /= torch.sqrt(torch.sum(col * col))
        if i + 1 < cols:
            rest = matrix[:, i + 1 :]
            rest -= torch.sum(col * rest, dim=0) * col


def _default_all_reduce(t: torch.Tensor) -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t)


class PowerSGDCompressor(Compressor):
    _state_fields = ("q_memory",)

    def __init__(self, rank=1, use_memory=False, world_size=1, all_reduce_fn=None):
        super().__init__()
        self.world_size = world_size
        self.q_memory = {}
        self.rank = rank
        self.use_memory = use_memory
        self.all_reduce_fn = all_reduce_fn or _default_all_reduce

    def compress(self, tensor, name):
        if tensor.dim() == 1:
            return [tensor], None
        shape = tensor.shape
        matrix = tensor.reshape(shape[0], -1)
        n, m = matrix.shape
        r = min(n, m, self.rank)
        if self.use_memory and name in self.q_memory and self.q_memory[name].shape == (m, r):
            q = self.q_memory[name]
        else:
            q = torch.randn(m, r, dtype=matrix.dtype, device=matrix.device)
            orthogonalize(q)
        p = matrix @ q
        self.all_reduce_fn(p)
        p = p / self.world_size
        orthogonalize(p)
        q = matrix.t() @ p
        self.all_reduce_fn(q)
        q = q / self.world_size
        if self.use_memory:
            self.q_memory[name] = q
        return [], (p, q, shape)

    def decompress(self, tensors, ctx):
        if ctx is None:
            (tensor,) = tensors
            return tensor
        p, q, shape = ctx
        return (p @ q.t()).view(shape)
