"""Momentum-corrected memory of Deep Gradient Compression.

Reference: ``grace_dl/dist/memory/dgc.py:7-39``: ``u = m*u + g``, ``v += u``,
compress ``v``; afterwards ``u`` and ``v`` are zeroed where the mask selected.
Attribute names follow the reference (``residuals`` is ``u``, ``gradients`` is
``v``) because they are the checkpoint keys.

Gradient clipping follows the working Horovod flavour
(``grace_dl/torch/memory/dgc.py:16-19``): clamp element-wise to
``+-sqrt(mean_over_ranks(sum g^2))``; the dist flavour of the reference divides
the ``None`` that ``dist.all_reduce`` returns and cannot run.
"""
import torch
from torch import distributed as dist

from ..core import Memory


class DgcMemory(Memory):
    _state_fields = ("residuals", "gradients")

    def __init__(self, momentum, gradient_clipping, world_size):
        self.gradient_clipping = gradient_clipping
        self.momentum = momentum
        self.world_size = world_size
        self.gradients = {}
        self.residuals = {}

    def _bound(self, tensor):
        """``sqrt(mean over ranks of sum g^2)`` as a 0-d tensor (one kernel on CUDA, ``csrc/memory.cu``)."""
        sq = None
        if tensor.is_cuda:
            from ..ops import memory as K

            sq = K.sum_squares(tensor)
            if sq is not None:
                sq = sq.to(torch.float32)
        if sq is None:
            sq = torch.sum(tensor * tensor)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(sq)
        return torch.sqrt(sq / self.world_size)

    def _clip(self, tensor):
        bound = self._bound(tensor)
        return torch.maximum(torch.minimum(tensor, bound), -bound)

    def compensate(self, tensor, name):
        if tensor.is_cuda and tensor.dtype == torch.float32:
            # momentum correction (and the clamp) as one kernel over g, u and v
            from ..ops import memory as K

            first = name not in self.residuals
            if first:
                self.residuals[name] = torch.empty_like(tensor)
                self.gradients[name] = torch.empty_like(tensor)
            u, v = self.residuals[name], self.gradients[name]
            bound = float(self._bound(tensor)) if self.gradient_clipping else float("inf")
            if u.shape == tensor.shape and K.dgc_compensate(tensor, u, v, self.momentum, bound, first):
                return v
            if first:
                del self.residuals[name], self.gradients[name]
        if self.gradient_clipping:
            tensor = self._clip(tensor)
        if name in self.residuals:
            self.residuals[name] = self.momentum * self.residuals[name] + tensor
        else:
            self.residuals[name] = tensor.clone()
        if name in self.gradients:
            self.gradients[name] = self.gradients[name] + self.residuals[name]
        else:
            self.gradients[name] = tensor.clone()
        return self.gradients[name]

    def update(self, tensor, name, compressor, tensor_compressed, ctx):
        shape, mask, _ = ctx
        u, v = self.residuals[name], self.gradients[name]
        if u.is_cuda and mask.is_cuda and u.data_ptr() != v.data_ptr():
            from ..ops import memory as K

            if K.dgc_mask(u, v, mask.reshape(-1)):
                return
        keep = ~mask.view(shape)
        self.residuals[name] = self.residuals[name] * keep
        self.gradients[name] = self.gradients[name] * keep
