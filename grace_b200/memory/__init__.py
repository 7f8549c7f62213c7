"""Error-feedback memories; import paths mirror ``grace_dl/dist/memory``."""
from .none import NoneMemory
from .residual import ResidualMemory
from .efsignsgd import EFSignSGDMemory
from .dgc import DgcMemory
from .powersgd import PowerSGDMemory

__all__ = ["NoneMemory", "ResidualMemory", "EFSignSGDMemory", "DgcMemory", "PowerSGDMemory"]
