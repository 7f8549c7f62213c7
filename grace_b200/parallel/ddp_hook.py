"""Communication hook for ``torch.nn.parallel.DistributedDataParallel``.

``register_grace_hook(ddp_model, grc)`` makes DDP hand every gradient bucket to
GRACE instead of all-reducing it.  GRACE compresses per *named parameter* (k,
norms and residuals are per tensor), so the hook builds, once per bucket index,
a segment table from ``bucket.parameters()`` and runs the fused exchange kernel
over the bucket on a high-priority side stream with a capped grid; the returned
future is tied to that stream (it completes on the device, nobody waits on the
host) and resolves to the bucket buffer holding the aggregated gradients.  With a library communicator (or on
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
        fused = hasattr(self.grc, "step_flat") and buf.is_cuda and buf.dtype == torch.float32 \
            and getattr(self.grc, "_kind", None) in ("sparse", "quant", "powersgd")
        if not fused:
            for p, g in zip(bucket.parameters(), bucket.gradients()):
                name = self.names.get(id(p), "param")
                g.copy_(self.grc.step(g, name).view_as(g))
            fut: torch.futures.Future = torch.futures.Future()
            fut.set_result(buf)
            return fut
        info = self._layout_for(bucket)
        layout = info["layout"]
        if self._stream is None:
            self._stream = torch.cuda.Stream(priority=-1)
        side = self._stream
        side.wait_stream(torch.cuda.current_stream())
        # A device-aware future: set_result() records an event on the stream that is current at that moment (the
        # side stream), and whoever consumes the future (DDP, when it finalises backward) makes ITS stream wait
        # for that event.  Neither the host nor the backward stream blocks here, so the exchange of this bucket
        # runs next to the backward kernels of the layers still to come.
        fut = torch.futures.Future(devices=[buf.device])
        limit = getattr(self.grc, "overlap_sms", None)
        with torch.cuda.stream(side):
            if info["aligned"] and buf.numel() == layout.total:
                self.grc.step_flat(buf, layout, sm_limit=limit)
            else:
                # DDP packs tensors back to back; the kernels want every tensor on a 128-element boundary:
                # one multi-tensor copy into an aligned staging buffer and one back
                stage = self._staging.get(info["key"])
                if stage is None:
                    flat = torch.zeros(layout.total, dtype=torch.float32, device=buf.device)
                    views = [flat[off:off + n] for off, n in zip(layout.offsets, layout.numels)]
                    stage = self._staging[info["key"]] = (flat, views)
                flat, views = stage
                # every gradient is a dense block of the bucket buffer (whatever its strides): address it there
                grads = [buf[off:off + n] for off, n in zip(info["offsets"], info["numels"])]
                torch._foreach_copy_(views, grads)
                self.grc.step_flat(flat, layout, sm_limit=limit)
                torch._foreach_copy_(grads, views)
            buf.record_stream(side)
            fut.set_result(buf)
        return fut


def register_grace_hook(ddp_model, grc):
    """Install GRACE as the gradient communication of a DDP-wrapped model."""
    hook = GraceDDPHook(grc, list(ddp_model.module.named_parameters()))

    def grace_comm_hook(state, bucket):  # DDP wants a plain function (it logs hook.__name__)
        return hook(state, bucket)

    ddp_model.register_comm_hook(None, grace_comm_hook)
    return hook
