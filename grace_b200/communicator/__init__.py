"""Communicators.  ``Allreduce``/``Allgather``/``Broadcast``/``AllToAll`` call
``torch.distributed`` (NCCL or gloo) and have the reference's semantics; they
are the baseline.  ``FusedExchange`` (``fused.py``) is the sm_100a path; ``HostExchange`` (``host.py``) runs the
same exchange protocol among CPU ranks in native code."""
from .allreduce import Allreduce
from .allgather import Allgather
from .broadcast import Broadcast
from .all_to_all import AllToAll

__all__ = ["Allreduce", "Allgather", "Broadcast", "AllToAll"]
