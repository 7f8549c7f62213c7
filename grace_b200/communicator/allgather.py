"""All-gather of the payload, then W decompressions and an aggregate.

Reference: ``grace_dl/dist/communicator/allgather.py:7-45`` and
``grace_dl/torch/communicator/allgather.py:7-53``.  Variable-size payloads
(Threshold, DGC, AdaQ, INCEPTIONN) first exchange their sizes, pad to the
per-component maximum and are sliced on receipt.  The size tensor stays on the
payload's device, so the path also runs on CPU ranks (the reference pins it to
``.cuda()``).
"""
import torch
from torch import distributed as dist

from ..core import Communicator
from . import _dist


class Allgather(Communicator):
    def _gather_same(self, t):
        out = [torch.empty_like(t) for _ in range(self.world_size)]
        work = dist.all_gather(out, t.contiguous(), async_op=True)
        return out, work, None

    def async_send(self, tensors, name):
        tensors = list(tensors)
        if not (_dist.active() and self.world_size > 1):
            return [([t], None, None) for t in tensors]
        if self.compressor.tensors_size_are_same:
            return [self._gather_same(t) for t in tensors]
        device = tensors[0].device
        local = torch.tensor([t.numel() for t in tensors], dtype=torch.int64, device=device)
        sizes = [torch.empty_like(local) for _ in range(self.world_size)]
        dist.all_gather(sizes, local)
        sizes = torch.stack(sizes).cpu()  # [W, n_payload]
        handles = []
        for j, t in enumerate(tensors):
            t = t.flatten()
            per_rank = sizes[:, j].tolist()
            widest = max(per_rank)
            padded = t.new_zeros(widest)
            padded[: t.numel()] = t
            out = [t.new_empty(widest) for _ in range(self.world_size)]
            work = dist.all_gather(out, padded, async_op=True)
            handles.append((out, work, per_rank))
        return handles

    def wait_receive(self, handles, ctx):
        columns = []
        for out, work, per_rank in handles:
            if work is not None:
                work.wait()
            if per_rank is not None:
                out = [o[:n] for o, n in zip(out, per_rank)]
            columns.append(out)
        decompressed = [self.compressor.decompress(list(parts), ctx) for parts in zip(*columns)]
        total = self.compressor.aggregate(decompressed)
        n = len(decompressed)
        return total / n if self.compressor.average else total
