"""Data-parallel integration: Horovod-style optimizer wrapper, DDP hook, flat
parameter buckets and the symmetric heap."""
from .optimizer import DistributedOptimizer  # noqa: F401


def __getattr__(name):
    if name == "FlatParams":
        from .flat import FlatParams

        return FlatParams
    if name == "register_grace_hook":
        from .ddp_hook import register_grace_hook

        return register_grace_hook
    if name == "SymmetricHeap":
        from .symm import SymmetricHeap

        return SymmetricHeap
    raise AttributeError(name)
