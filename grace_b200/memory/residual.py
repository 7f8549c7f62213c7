"""Residual (error-feedback) memory.

Reference: ``grace_dl/dist/memory/residual.py:4-20``:
``acc = beta*residual + gamma*g`` once a residual exists (the very first step
uses ``g`` unscaled), ``residual = acc - decompress(compress(acc))``.
"""
from ..core import Memory


class ResidualMemory(Memory):
    _state_fields = ("residuals",)

    def __init__(self, beta=1.0, gamma=1.0):
        self.residuals = {}
        self.beta = beta
        self.gamma = gamma

    def compensate(self, tensor, name):
        if name in self.residuals:
            tensor = self.beta * self.residuals[name] + self.gamma * tensor
        return tensor

    def update(self, tensor, name, compressor, tensor_compressed, ctx):
        self.residuals[name] = tensor - compressor.decompress(tensor_compressed, ctx)
