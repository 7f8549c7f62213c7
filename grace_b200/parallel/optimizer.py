"""Horovod-style ``DistributedOptimizer`` without Horovod.

What a user of the reference's patched ``horovod/torch/optimizer.py:35-277,
451-519`` relies on, and gets here:

* ``DistributedOptimizer(opt, grace=grc, named_parameters=...)`` returns an
  object whose class is a subclass of ``type(opt)`` carrying its name
  (``state_dict`` is the wrapped optimizer's own);
* parameters without a name are called ``allreduce.noname.<i>``; a
  ``named_parameters`` that is not a sequence of pairs, repeats a name or
  leaves a parameter out is rejected with ``ValueError``;
* when a gradient has been accumulated ``backward_passes_per_step`` times the
  exchange of that gradient starts, inside backward
  (``grace.send_step(p.grad, name)``), and ``synchronize()`` finishes it
  (``p.grad.set_(grace.receive_step(handle, ctx))``), also starting the
  exchanges whose hook never ran;
* ``step()`` synchronises first unless called under ``skip_synchronize()``,
  and warns when ``synchronize()`` had already been called without it;
* ``zero_grad()`` between ``backward()`` and ``step()`` raises;
  ``load_state_dict`` and ``set_backward_passes_per_step`` re-arm the counters;
* ``num_groups > 0`` or ``op != Average`` take GRACE out of the path
  (plain all-reduce); with ``num_groups`` the parameters are split into that
  many groups and each group is reduced by ONE all-reduce of its flattened
  gradients, started when the last gradient of the group is ready.

How it is built here: every parameter has a ledger entry (name, countdown,
in-flight ticket); the entries point to an optional *bucket* (a range of a
``FlatParams`` buffer exchanged by one fused kernel) or *group* (plain
all-reduce of several tensors at once).  Bucket exchanges run on a
high-priority side stream with a capped grid while backward continues;
``synchronize()`` only makes the compute stream wait for their events.
"""
from __future__ import annotations

import os
import warnings
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch
from torch import distributed as dist

Average, Sum = "average", "sum"


def _world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


class _Entry:
    """Ledger line of one parameter."""

    __slots__ = ("param", "name", "countdown", "ticket", "ctx", "armed", "group")

    def __init__(self, param, name, passes):
        self.param, self.name = param, name
        self.countdown = passes      # backward passes left before the exchange starts
        self.ticket = None           # what send_step / the plain all-reduce handed back
        self.ctx = None
        self.armed = False           # a backward pass touched this parameter since the last synchronize
        self.group = None


class _Group:
    """Parameters whose gradients travel in one plain all-reduce (``num_groups``)."""

    def __init__(self, index: int, entries: List[_Entry]):
        self.index, self.entries = index, entries
        self.waiting = len(entries)
        self.flat = None
        self.work = None

    def rearm(self):
        self.waiting, self.flat, self.work = len(self.entries), None, None


def _validated_names(param_groups, named_parameters) -> List[tuple]:
    """(name, parameter) pairs for every parameter of the optimizer, or ValueError."""
    params = [p for g in param_groups for p in g["params"]]
    if named_parameters is None:
        pairs = []
        for g in param_groups:
            pairs.extend(("allreduce.noname.%s" % i, p) for i, p in enumerate(g["params"]))
        return pairs
    pairs = list(named_parameters)
    if not all(isinstance(kv, tuple) for kv in pairs):
        raise ValueError("named_parameters should be a sequence of tuples (name, parameter), "
                         "usually produced by model.named_parameters().")
    repeated = _DistributedMixin.find_duplicates([k for k, _ in pairs])
    if repeated:
        raise ValueError("Parameter names in named_parameters must be unique. Found duplicates: %s"
                         % ", ".join(sorted(repeated)))
    covered = {id(p) for _, p in pairs}
    missing = [str(id(p)) for p in params if id(p) not in covered]
    if missing:
        raise ValueError("named_parameters was specified, but one or more model parameters were not named. "
                         "Python object ids: %s" % ", ".join(missing))
    return pairs


class _DistributedMixin:
    """Methods mixed in front of the user's optimizer class (see ``DistributedOptimizer``)."""

    # ---- set-up --------------------------------------------------------------
    def _grace_setup(self, named_parameters, grace, compression, backward_passes_per_step, op,
                     gradient_predivide_factor, num_groups, flat, always_hook):
        self._grace = grace
        self._compression = compression
        self.backward_passes_per_step = backward_passes_per_step
        self.op = op
        self.gradient_predivide_factor = gradient_predivide_factor
        self._num_groups = int(num_groups)
        self._flat = flat
        self._ledger: Dict[torch.nn.Parameter, _Entry] = {}
        for name, p in sorted(_validated_names(self.param_groups, named_parameters), key=lambda kv: kv[0]):
            self._ledger[p] = _Entry(p, name, backward_passes_per_step)
        self._groups: List[_Group] = []
        self._bucket_events = {}
        self._side_stream = None
        self._hook_handles = []
        self._synchronized = False
        self._should_synchronize = True
        self._in_flight = False       # a backward pass ran since the last synchronize
        self.trace_overlap = False    # True: keep (bucket, start event, end event, launched from a hook) per exchange
        self.overlap_log = []         # ... of the current step, with timing events (see tests/test_gpu_pipeline.py)
        if _world_size() > 1 or always_hook or os.environ.get("GRACE_ELASTIC") == "1":
            self._install_hooks()

    @property
    def _parameter_names(self):
        return {p: e.name for p, e in self._ledger.items()}

    @staticmethod
    def find_duplicates(lst):
        counts: Dict[object, int] = {}
        for item in lst:
            counts[item] = counts.get(item, 0) + 1
        return {item for item, c in counts.items() if c > 1}

    def _uses_grace(self) -> bool:
        return self._grace is not None and self._num_groups == 0 and self.op == Average

    def _bucketed(self) -> bool:
        return (self._uses_grace() and self._flat is not None and hasattr(self._grace, "step_flat")
                and self._flat.flat_g.is_cuda)

    def _trainable(self) -> List[torch.nn.Parameter]:
        return [p for g in self.param_groups for p in g["params"] if p.requires_grad]

    def _install_hooks(self):
        trainable = self._trainable()
        for p in trainable:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            if hasattr(p, "register_post_accumulate_grad_hook"):
                self._hook_handles.append(p.register_post_accumulate_grad_hook(self._on_gradient))
            else:   # older torch: the AccumulateGrad node itself
                node = p.expand_as(p).grad_fn.next_functions[0][0]
                node.register_hook(lambda *_, _p=p: self._on_gradient(_p))
                self._hook_handles.append(node)
        if self._num_groups > 0:
            # the same split on every rank: by name, into num_groups runs of (nearly) equal length
            ordered = sorted(trainable, key=lambda p: self._ledger[p].name)
            n, g = len(ordered), max(1, min(self._num_groups, len(ordered)))
            cuts = [round(i * n / g) for i in range(g + 1)]
            for i in range(g):
                entries = [self._ledger[p] for p in ordered[cuts[i]:cuts[i + 1]]]
                if entries:
                    grp = _Group(len(self._groups), entries)
                    for e in entries:
                        e.group = grp
                    self._groups.append(grp)
        if self._bucketed():
            for b in self._flat.buckets:
                b.pending = len(b.layout.names)
            if hasattr(self._grace, "prepare_layouts"):
                self._grace.prepare_layouts([b.layout for b in self._flat.buckets], self._flat.flat_g.device)
        elif self._uses_grace() and hasattr(self._grace, "prepare"):
            # plans (symmetric memory, flags) exist before the first backward pass fires any hook
            self._grace.prepare([(self._ledger[p].name, p.grad) for p in trainable if p.grad is not None])

    # ---- re-arming -------------------------------------------------------------
    def _rearm(self, entries=None):
        for e in (self._ledger.values() if entries is None else entries):
            e.countdown, e.ticket, e.ctx, e.armed = self.backward_passes_per_step, None, None, False

    def load_state_dict(self, *args, **kwargs):
        self._rearm()
        for grp in self._groups:
            grp.rearm()
        self._in_flight = False
        self._synchronized = False
        self._should_synchronize = True
        super().load_state_dict(*args, **kwargs)

    def set_backward_passes_per_step(self, passes):
        self.backward_passes_per_step = passes
        for e in self._ledger.values():
            e.countdown = passes

    # ---- launches ----------------------------------------------------------------
    def _comm_stream(self):
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(priority=-1)
        return self._side_stream

    def _launch_bucket(self, bucket, overlapped: bool, from_hook: bool = True):
        """One fused exchange for the whole bucket, on the side stream.  ``overlapped``: backward is still
        running, so the kernel takes a capped share of the SMs (``grace.overlap_sms``).  ``overlap_log`` entries:
        ``(bucket, start event, end event, launched from a gradient hook, capped)``."""
        side = self._comm_stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            if self.trace_overlap:
                start = torch.cuda.Event(enable_timing=True)
                start.record(side)
            g = self._flat.grad_view(bucket)
            if self.gradient_predivide_factor != 1.0:
                g.div_(self.gradient_predivide_factor)
            limit = getattr(self._grace, "overlap_sms", None) if overlapped else None
            if limit is not None:
                self._grace.step_flat(g, bucket.layout, sm_limit=limit)
            else:
                self._grace.step_flat(g, bucket.layout)
            ev = torch.cuda.Event(enable_timing=self.trace_overlap)
            ev.record(side)
            if self.trace_overlap:
                self.overlap_log.append((bucket.index, start, ev, from_hook, overlapped))
        self._bucket_events[bucket.index] = ev

    def _plain_allreduce(self, tensor):
        """(tensor on the wire, work, wire context) of an averaged / summed all-reduce without GRACE."""
        work = wire_ctx = None
        if _world_size() > 1:
            if self.op == Average:
                tensor.div_(_world_size())
            if self._compression is not None:      # Horovod's wire-format compression (none / fp16)
                tensor, wire_ctx = self._compression.compress(tensor)
            work = dist.all_reduce(tensor, async_op=True)
        return tensor, work, wire_ctx

    def _launch_entry(self, e: _Entry):
        if self._uses_grace():
            e.ticket, e.ctx = self._grace.send_step(e.param.grad, e.name)
            return
        if e.group is not None:
            grp = e.group
            grp.waiting -= 1
            e.ticket = ("group", grp.index)
            if grp.waiting == 0:
                grp.flat = torch._utils._flatten_dense_tensors([x.param.grad for x in grp.entries])
                grp.flat, grp.work, _ = self._plain_allreduce(grp.flat)
            return
        tensor, work, wire_ctx = self._plain_allreduce(e.param.grad)
        e.ticket, e.ctx = ("plain", tensor, work), wire_ctx

    def _on_gradient(self, p):
        e = self._ledger[p]
        if e.ticket is not None and e.countdown <= 0:
            raise AssertionError(
                "Gradients were computed more than backward_passes_per_step times before call to step(). "
                "Increase backward_passes_per_step to accumulate gradients locally.")
        assert not p.grad.requires_grad
        e.armed = True
        self._in_flight = True
        e.countdown -= 1
        if e.countdown != 0:
            return
        if self._bucketed():
            bucket = self._flat.bucket_of[e.name]
            bucket.pending -= 1
            e.ticket = ("bucket", bucket.index)
            if bucket.pending == 0:
                # the last bucket of a step has (almost) nothing of backward left to share the SMs with: full width
                last = len(self._bucket_events) == len(self._flat.buckets) - 1
                self._launch_bucket(bucket, overlapped=not last)
        else:
            self._launch_entry(e)

    # ---- synchronisation ---------------------------------------------------------------
    def synchronize(self):
        entries = [self._ledger[p] for p in self._trainable() if p in self._ledger]
        if self._bucketed():
            for b in self._flat.buckets:
                if b.index not in self._bucket_events:
                    self._launch_bucket(b, overlapped=False, from_hook=False)   # backward is over: nothing left to share the SMs with
            cur = torch.cuda.current_stream()
            for ev in self._bucket_events.values():
                cur.wait_event(ev)
            self._bucket_events.clear()
            for b in self._flat.buckets:
                b.pending = len(b.layout.names)
        else:
            for e in entries:
                if e.ticket is None:     # hook never ran, or the countdown has not reached zero yet
                    self._launch_entry(e)
            for grp in self._groups:
                if grp.work is not None:
                    grp.work.wait()
                if grp.flat is not None:
                    flat = grp.flat
                    if self._compression is not None and grp.work is not None:
                        flat = self._compression.decompress(flat, None)
                    grads = [x.param.grad for x in grp.entries]
                    for g, piece in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
                        g.copy_(piece)
                grp.rearm()
            for e in entries:
                t = e.ticket
                if isinstance(t, tuple) and t and t[0] == "group":
                    continue
                if isinstance(t, tuple) and len(t) == 3 and t[0] == "plain":
                    _, tensor, work = t
                    if work is not None:
                        work.wait()
                    output = tensor
                    if self._compression is not None and work is not None:
                        output = self._compression.decompress(tensor, e.ctx)
                else:
                    output = self._grace.receive_step(t, e.ctx)
                if output.data_ptr() != e.param.grad.data_ptr():
                    e.param.grad.set_(output.to(e.param.grad.dtype).view(e.param.grad.shape))
        self._rearm(entries)
        self._in_flight = False
        self._synchronized = True
        if self.trace_overlap:
            self.last_overlap_log, self.overlap_log = self.overlap_log, []

    @contextmanager
    def skip_synchronize(self):
        self._should_synchronize = False
        try:
            yield
        finally:
            self._should_synchronize = True

    def step(self, closure=None):
        if self._should_synchronize:
            if self._synchronized:
                warnings.warn("optimizer.step() called without optimizer.skip_synchronize() context after "
                              "optimizer.synchronize(). This can cause training slowdown. You may want to consider "
                              "using optimizer.skip_synchronize() context if you use optimizer.synchronize() in your code.")
            self.synchronize()
        self._synchronized = False
        return super().step(closure)

    def zero_grad(self, *args, **kwargs):
        if self._in_flight:
            raise AssertionError("optimizer.zero_grad() was called after loss.backward() but before optimizer.step() "
                                 "or optimizer.synchronize(). This is prohibited as it can cause a race condition.")
        if self._flat is not None or self._hook_handles:
            kwargs["set_to_none"] = False  # gradients are exchanged in place; keep their storage
            args = ()
        return super().zero_grad(*args, **kwargs)


def DistributedOptimizer(optimizer, grace=None, named_parameters=None, compression=None, backward_passes_per_step=1,
                         op=Average, gradient_predivide_factor=1.0, num_groups=0, flat=None, always_hook=False):
    """Wrap ``optimizer`` so that gradients are exchanged through ``grace``.

    Same call as ``hvd.DistributedOptimizer(optimizer, grace=..., named_parameters=...)`` of the reference
    (``patch_files/horovod/torch/optimizer.py:451-519``).  The result shares the wrapped optimizer's parameter
    groups, state and every attribute it had set up (flat buffers and momentum of ``FusedSGD``, ...).
    ``flat=FlatParams(...)`` with a ``FusedExchange`` switches to bucket-wise exchanges.
    """
    if gradient_predivide_factor != 1.0 and op != Average:
        raise ValueError("gradient_predivide_factor not supported with op != Average")
    base = optimizer.__class__
    cls = type(base.__name__, (_DistributedMixin, base), {})
    obj = cls.__new__(cls)
    obj.__dict__.update(optimizer.__dict__)
    if flat is None:
        flat = getattr(optimizer, "flat", None)
    obj._grace_setup(named_parameters, grace, compression, backward_passes_per_step, op, gradient_predivide_factor,
                     num_groups, flat, always_hook)
    return obj
