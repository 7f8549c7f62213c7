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

    def _clip(self, tensor):
        sq = torch.sum(tensor * tensor)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(sq)
        bound = torch.sqrt(sq / self.world_size)
        return torch.maximum(torch.minimum(tensor, bound), -bound)

    def compensate(self, tensor, name):
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
        keep = ~mask.view(shape)
        self.residuals[name] = self.residuals[name] * keep
        self.gradients[name] = self.gradients[name] * keep
