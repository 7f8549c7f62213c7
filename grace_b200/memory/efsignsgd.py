"""Memory of EF-signSGD.  Reference: ``grace_dl/dist/memory/efsignsgd.py:4-19``:
``acc = residual + lr*g`` once a residual exists."""
from ..core import Memory


class EFSignSGDMemory(Memory):
    _state_fields = ("residuals",)

    def __init__(self, lr):
        self.residuals = {}
        self.learning_rate = lr

    def compensate(self, tensor, name):
        if name in self.residuals:
            tensor = self.residuals[name] + self.learning_rate * tensor
        return tensor

    def update(self, tensor, name, compressor, tensor_compressed, ctx):
        self.residuals[name] = tensor - compressor.decompress(tensor_compressed, ctx)
