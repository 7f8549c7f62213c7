"""W broadcasts (root = 0..W-1) of every payload tensor.

Reference: ``grace_dl/dist/communicator/broadcast.py:7-33``.  ``rank`` defaults
to the process group's rank so that ``grace_from_params`` can build this class
(the reference factory omits the argument and cannot).
"""
import torch
from torch import distributed as dist

from ..core import Communicator
from . import _dist


class Broadcast(Communicator):
    def __init__(self, compressor, memory, world_size, rank=None):
        super().__init__(compressor, memory, world_size)
        if rank is None:
            rank = dist.get_rank() if _dist.active() else 0
        self.rank = rank

    def async_send(self, tensors, name):
        if not self.compressor.tensors_size_are_same:
            raise NotImplementedError("Broadcast needs equally sized payloads on every rank")
        tensors = list(tensors)
        if not (_dist.active() and self.world_size > 1):
            return [[(t, None)] for t in tensors]
        handles = []
        for t in tensors:
            per_root = []
            for root in range(self.world_size):
                buf = t.contiguous() if root == self.rank else torch.empty_like(t)
                per_root.append((buf, dist.broadcast(buf, root, async_op=True)))
            handles.append(per_root)
        return handles

    def wait_receive(self, handles, ctx):
        columns = []
        for per_root in handles:
            bufs = []
            for buf, work in per_root:
                if work is not None:
                    work.wait()
                bufs.append(buf)
            columns.append(bufs)
        decompressed = [self.compressor.decompress(list(parts), ctx) for parts in zip(*columns)]
        total = self.compressor.aggregate(decompressed)
        n = len(decompressed)
        return total / n if self.compressor.average else total
