"""All-reduce of the payload tensors (library collective).

Reference: ``grace_dl/dist/communicator/allreduce.py:6-13`` and the handle
based ``grace_dl/torch/communicator/allreduce.py:5-15``.  Meaningful for
payloads that are linear in the gradient: none, fp16, randomk, powersgd.
"""
from torch import distributed as dist

from ..core import Communicator
from . import _dist


class Allreduce(Communicator):
    def async_send(self, tensors, name):
        handles = []
        for t in tensors:
            work = None
            if _dist.active() and self.world_size > 1:
                work = dist.all_reduce(t, async_op=True)
            handles.append((t, work))
        return handles

    def wait_receive(self, handles, ctx):
        reduced = []
        for t, work in handles:
            if work is not None:
                work.wait()
            if self.compressor.average:
                t = t / self.world_size if not t.is_floating_point() else t.div_(self.world_size)
            reduced.append(t)
        return self.compressor.decompress(reduced, ctx)
