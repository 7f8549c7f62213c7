"""grace_b200: gradient compression for data-parallel training, written for
NVIDIA B200 (sm_100a).

Public surface (same names as the reference's ``grace_dl.dist`` and
``grace_dl.torch`` packages):

* ``Memory`` / ``Compressor`` / ``Communicator`` base classes,
* ``grace_from_params`` factory,
* ``grace_b200.compressor``, ``grace_b200.memory``, ``grace_b200.communicator``,
* ``grace_b200.parallel``: ``DistributedOptimizer`` (Horovod style), DDP
  communication hook, flat gradient buckets,
* ``grace_b200.optim.FusedSGD``,
* ``grace_b200.ops``: the CUDA kernels.
"""
from .core import Communicator, Compressor, Memory
from .helper import grace_from_params

__version__ = "0.1.0"
__all__ = ["Communicator", "Compressor", "Memory", "grace_from_params", "__version__"]
