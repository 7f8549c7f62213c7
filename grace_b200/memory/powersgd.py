"""Residual memory for PowerSGD.

Reference: ``grace_dl/dist/memory/powersgd.py:6-37``: 1-D tensors are left
alone; matrices get last step's residual added before the projections and
``residual = M - P Q^T`` afterwards.  The reference also overwrites the shared
``q_memory[name]`` with fresh noise on every ``compensate`` which defeats the
warm start; this class leaves ``q_memory`` to the compressor.
"""
from ..core import Memory


class PowerSGDMemory(Memory):
    _state_fields = ("residuals",)

    def __init__(self, q_memory, compress_rank=1):
        self.compress_rank = compress_rank
        self.q_memory = q_memory
        self.residuals = {}

    def compensate(self, tensor, name):
        if tensor.dim() == 1:
            return tensor
        if name in self.residuals:
            tensor = tensor + self.residuals[name]
        return tensor

    def update(self, tensor, name, compressor, tensor_compressed, ctx):
        if ctx is None:
            return
        self.residuals[name] = tensor - compressor.decompress(tensor_compressed, ctx)
