"""Communication hook for ``torch.nn.parallel.DistributedDataParallel``.

``register_grace_hook(ddp_model, grc)`` makes DDP hand every gradient bucket to
GRACE instead of all-reducing it.  GRACE compresses per *named parameter* (k,
norms and residuals are per tensor), so the hook builds, once per bucket index,
a segment table from ``bucket.parameters()`` and runs the fused exchange kernel
over the bucket on a side stream; the returned future resolves to the bucket
buffer holding the aggregated gradients.  With a library communicator (or on
CPU) the hook falls back to ``grc.step`` per parameter.  DDP re-partitions its
buckets once, after the first iteration; error-feedback state collected during
that first iteration belongs to the old partition and is not carried over.

The reference has no DDP integration: its "DDP" example is a Python loop over
``model.named_parameters()`` after ``backward()`` with no overlap
(``examples/dist/CIFAR10-dawndist/core.py:203-206``).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops.exchange import ALIGN_ELEMS, FlatLayout


class GraceDDPHook:
    def __init__(self, grc, named_parameters):
        self.grc = grc
        self.names: Dict[int, str] = {id(p): n for n, p in named_parameters}
        self._layouts = {}
        self._stream = None
        self._staging = {}

    def _layout_for(self, bucket):
        idx = bucket.index()
        params = bucket.parameters()
        grads = bucket.gradients()
        # DDP re-partitions its buckets after the first iteration: the cache key is the bucket's content
        key = (idx, tuple(id(p) for p in params))
        if key in self._layouts:
            return self._layouts[key]
        base = bucket.buffer().data_ptr()
        names, numels, offsets = [], [], []
        aligned = base % 16 == 0
        for p, g in zip(params, grads):
            names.append(self.names.get(id(p), "param.%d.%d" % (idx, len(names))))
            numels.append(g.numel())
            off = (g.data_ptr() - base) // 4
            offsets.append(off)
            aligned = aligned and off % ALIGN_ELEMS == 0
        total = (bucket.buffer().numel() + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
        layout = FlatLayout(names, numels, offsets, total) if aligned else FlatLayout(names, numels)
        layout.shapes = [tuple(p.shape) for p in params]
        info = dict(names=names, numels=numels, offsets=offsets, aligned=aligned, layout=layout)
        info["key"] = key
        self._layouts[key] = info
        return info

    def __call__(self, state, bucket):  # returns torch.futures.Future[torch.Tensor]
        buf = bucket.buffer()
        fut: torch.futures.Future = torch.futures.Future()
        fused = hasattr(self.grc, "step_flat") and buf.is_cuda and buf.dtype == torch.float32 \
            and getattr(self.grc, "_kind", None) in ("sparse", "quant", "powersgd")
        if not fused:
            for p, g in zip(bucket.parameters(), bucket.gradients()):
                name = self.names.get(id(p), "param")
                g.copy_(self.grc.step(g, name).view_as(g))
            fut.set_result(buf)
            return fut
        info = self._layout_for(bucket)
        layout = info["layout"]
        if self._stream is None:
            self._stream = torch.cuda.Stream(priority=-1)
        side = self._stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            if info["aligned"] and buf.numel() == layout.total:
                self.grc.step_flat(buf, layout)
            else:
                # DDP packs tensors back to back: stage into an aligned buffer
                stage = self._staging.get(info["key"])
                if stage is None:
                    stage = torch.zeros(layout.total, dtype=torch.float32, device=buf.device)
                    self._staging[info["key"]] = stage
                for g, off, n in zip(bucket.gradients(), layout.offsets, layout.numels):
                    stage[off:off + n].copy_(g.reshape(-1))
                self.grc.step_flat(stage, layout)
                for g, off, n in zip(bucket.gradients(), layout.offsets, layout.numels):
                    g.copy_(stage[off:off + n].view_as(g))
            ev = torch.cuda.Event()
            ev.record(side)
        torch.cuda.current_stream().wait_event(ev)
        fut.set_result(buf)
        return fut


def register_grace_hook(ddp_model, grc):
    """Install GRACE as the gradient communication of a DDP-wrapped model."""
    hook = GraceDDPHook(grc, list(ddp_model.module.named_parameters()))

    def grace_comm_hook(state, bucket):  # DDP wants a plain function (it logs hook.__name__)
        return hook(state, bucket)

    ddp_model.register_comm_hook(None, grace_comm_hook)
    return hook
