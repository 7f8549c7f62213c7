"""Residual (error-feedback) memory.

Reference: ``grace_dl/dist/memory/residual.py:4-20``:
``acc = beta*residual + gamma*g`` once a residual exists (the very first step
uses ``g`` unscaled), ``residual = acc - decompress(compress(acc))``.

On CUDA tensors both halves are single streaming kernels (``csrc/memory.cu``);
for the sparse codecs the residual is the accumulator with the transmitted
positions zeroed, so nothing dense is decompressed.
"""
from ..core import Memory
from ._cuda import sparse_payload, state_like


class ResidualMemory(Memory):
    _state_fields = ("residuals",)

    def __init__(self, beta=1.0, gamma=1.0):
        self.residuals = {}
        self.beta = beta
        self.gamma = gamma

    def compensate(self, tensor, name):
        residual = self.residuals.get(name)
        if residual is None:
            return tensor
        if tensor.is_cuda:
            from ..ops import memory as K

            out = K.residual_compensate(tensor, state_like(residual, tensor), self.beta, self.gamma)
            if out is not None:
                return out
        return self.beta * residual + self.gamma * tensor

    def update(self, tensor, name, compressor, tensor_compressed, ctx):
        if tensor.is_cuda:
            from ..ops import memory as K

            indices = sparse_payload(compressor, tensor_compressed)
            out = K.sparse_residual(tensor, indices) if indices is not None else None
            if out is None and indices is None:
                out = K.residual_update(tensor, compressor.decompress(tensor_compressed, ctx))
            if out is not None:
                self.residuals[name] = out
                return
        self.residuals[name] = tensor - compressor.decompress(tensor_compressed, ctx)
