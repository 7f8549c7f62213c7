"""Memory of EF-signSGD.  Reference: ``grace_dl/dist/memory/efsignsgd.py:4-19``:
``acc = residual + lr*g`` once a residual exists.  On CUDA tensors each half is one
streaming kernel (``csrc/memory.cu``)."""
from ..core import Memory
from ._cuda import state_like


class EFSignSGDMemory(Memory):
    _state_fields = ("residuals",)

    def __init__(self, lr):
        self.residuals = {}
        self.learning_rate = lr

    def compensate(self, tensor, name):
        residual = self.residuals.get(name)
        if residual is None:
            return tensor
        if tensor.is_cuda:
            from ..ops import memory as K

            out = K.residual_compensate(tensor, state_like(residual, tensor), 1.0, self.learning_rate)
            if out is not None:
                return out
        return residual + self.learning_rate * tensor

    def update(self, tensor, name, compressor, tensor_compressed, ctx):
        decompressed = compressor.decompress(tensor_compressed, ctx)
        if tensor.is_cuda:
            from ..ops import memory as K

            out = K.residual_update(tensor, decompressed)
            if out is not None:
                self.residuals[name] = out
                return
        self.residuals[name] = tensor - decompressed
