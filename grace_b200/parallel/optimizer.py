"""Horovod-style ``DistributedOptimizer`` without Horovod.

Contract reproduced from the reference's patched
``horovod/torch/optimizer.py:35-277,451-519``:

* the returned object is an instance of a dynamically created subclass of the
  user's optimizer class (``state_dict`` is the wrapped optimizer's own);
* names default to ``allreduce.noname.<i>``; tuples, duplicate names and
  unnamed parameters are rejected;
* a hook on every parameter's gradient accumulation decrements a per-parameter
  delay counter (``backward_passes_per_step``) and, at zero, launches
  ``grace.send_step(p.grad, name)`` so the exchange overlaps with the rest of
  backward;
* ``synchronize()`` launches what never fired, then
  ``p.grad.set_(grace.receive_step(handle, ctx))``;
* ``step()`` synchronises unless inside ``skip_synchronize()`` and warns on a
  redundant ``synchronize()``; ``zero_grad()`` refuses to run with exchanges in
  flight; ``load_state_dict`` and ``set_backward_passes_per_step`` reset the
  counters.

B200 additions: with ``flat=FlatParams(...)`` and a ``FusedExchange`` the hooks
work per *bucket*: when the last gradient of a bucket has been accumulated the
whole bucket is exchanged by one fused kernel on a high-priority side stream,
and ``synchronize()`` only makes the compute stream wait for those launches.
``grace=None`` gives a plain averaged all-reduce.
"""
from __future__ import annotations

import os
import warnings
from contextlib import contextmanager

import torch
from torch import distributed as dist

Average, Sum = "average", "sum"


def _world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


class _DistributedOptimizer(torch.optim.Optimizer):
    def __init__(self, params, named_parameters, grace, compression=None, backward_passes_per_step=1, op=Average,
                 gradient_predivide_factor=1.0, num_groups=0, flat=None, always_hook=False):
        super(self.__class__, self).__init__(params)
        self._grace = grace
        self._compression = compression
        if named_parameters is not None:
            named_parameters = list(named_parameters)
        else:
            named_parameters = [("allreduce.noname.%s" % i, v)
                                for group in self.param_groups for i, v in enumerate(group["params"])]
        if any(not isinstance(p, tuple) for p in named_parameters):
            raise ValueError("named_parameters should be a sequence of tuples (name, parameter), "
                             "usually produced by model.named_parameters().")
        dups = self.find_duplicates([k for k, _ in named_parameters])
        if dups:
            raise ValueError("Parameter names in named_parameters must be unique. Found duplicates: %s"
                             % ", ".join(sorted(dups)))
        all_ids = {id(v) for group in self.param_groups for v in group["params"]}
        named_ids = {id(v) for _, v in named_parameters}
        unnamed = all_ids - named_ids
        if unnamed:
            raise ValueError("named_parameters was specified, but one or more model parameters were not named. "
                             "Python object ids: %s" % ", ".join(str(i) for i in unnamed))
        ordered = sorted(named_parameters, key=lambda kv: kv[0])
        self._parameter_names = {v: k for k, v in ordered}
        self.backward_passes_per_step = backward_passes_per_step
        self._allreduce_delay = {v: backward_passes_per_step for _, v in ordered}
        self.op = op
        self.gradient_predivide_factor = gradient_predivide_factor
        self._num_groups = num_groups
        self._handles = {}
        self._grad_accs = []
        self._requires_update = set()
        self._synchronized = False
        self._should_synchronize = True
        self._flat = flat
        self._bucket_events = {}
        self._side_stream = None
        if _world_size() > 1 or always_hook or os.environ.get("GRACE_ELASTIC") == "1":
            self._register_hooks()

    # -- bookkeeping --------------------------------------------------------
    @staticmethod
    def find_duplicates(lst):
        seen, dups = set(), set()
        for el in lst:
            if el in seen:
                dups.add(el)
            seen.add(el)
        return dups

    def load_state_dict(self, *args, **kwargs):
        self._handles = {}
        self._synchronized = False
        self._should_synchronize = True
        for p in self._allreduce_delay:
            self._allreduce_delay[p] = self.backward_passes_per_step
        super(self.__class__, self).load_state_dict(*args, **kwargs)

    def set_backward_passes_per_step(self, passes):
        self.backward_passes_per_step = passes
        for p in self._allreduce_delay:
            self._allreduce_delay[p] = passes

    # -- hooks ----------------------------------------------------------------
    def _register_hooks(self):
        for group in self.param_groups:
            for p in group["params"]:
                if not p.requires_grad:
                    continue
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
                self._requires_update.add(p)
                if hasattr(p, "register_post_accumulate_grad_hook"):
                    self._grad_accs.append(p.register_post_accumulate_grad_hook(self._make_hook(p)))
                else:  # older torch: hook the AccumulateGrad node as Horovod does
                    acc = p.expand_as(p).grad_fn.next_functions[0][0]
                    acc.register_hook(self._make_hook(p))
                    self._grad_accs.append(acc)
        if self._bucketed():
            for b in self._flat.buckets:
                b.pending = len(b.layout.names)

    def _bucketed(self) -> bool:
        return self._flat is not None and hasattr(self._grace, "step_flat") and self._flat.flat_g.is_cuda

    def _comm_stream(self):
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(priority=-1)
        return self._side_stream

    def _launch_bucket(self, bucket):
        side = self._comm_stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            g = self._flat.grad_view(bucket)
            if self.gradient_predivide_factor != 1.0:
                g.div_(self.gradient_predivide_factor)
            self._grace.step_flat(g, bucket.layout)
            ev = torch.cuda.Event()
            ev.record(side)
        self._bucket_events[bucket.index] = ev

    def _allreduce_grad_async(self, p):
        name = self._parameter_names.get(p)
        tensor = p.grad
        if self._grace is not None and self._num_groups == 0 and self.op == Average:
            return self._grace.send_step(tensor, name)
        work = None
        wire_ctx = None
        if _world_size() > 1:
            if self.op == Average:
                tensor.div_(_world_size())
            if self._compression is not None:      # Horovod's wire-format compression (none / fp16)
                tensor, wire_ctx = self._compression.compress(tensor)
            work = dist.all_reduce(tensor, async_op=True)
        return ("plain", tensor, work), wire_ctx

    def _make_hook(self, p):
        def hook(*ignore):
            if p in self._handles and self._handles[p][0] is not None:
                if self._allreduce_delay[p] <= 0:
                    raise AssertionError(
                        "Gradients were computed more than backward_passes_per_step times before call to step(). "
                        "Increase backward_passes_per_step to accumulate gradients locally.")
            assert not p.grad.requires_grad
            assert self._allreduce_delay[p] > 0
            handle, ctx = None, None
            self._allreduce_delay[p] -= 1
            if self._allreduce_delay[p] == 0:
                if self._bucketed():
                    bucket = self._flat.bucket_of[self._parameter_names[p]]
                    bucket.pending -= 1
                    handle = ("bucket", bucket.index)
                    if bucket.pending == 0:
                        self._launch_bucket(bucket)
                else:
                    handle, ctx = self._allreduce_grad_async(p)
            self._handles[p] = (handle, ctx)

        return hook

    # -- synchronisation --------------------------------------------------------
    def synchronize(self):
        missing = self._requires_update - set(self._handles.keys())
        if self._bucketed():
            for p in missing:
                self._handles[p] = (("bucket", self._flat.bucket_of[self._parameter_names[p]].index), None)
            for b in self._flat.buckets:
                if b.index not in self._bucket_events:
                    self._launch_bucket(b)
            cur = torch.cuda.current_stream()
            for ev in self._bucket_events.values():
                cur.wait_event(ev)
            self._bucket_events.clear()
            for b in self._flat.buckets:
                b.pending = len(b.layout.names)
            for p in self._handles:
                self._allreduce_delay[p] = self.backward_passes_per_step
            self._handles.clear()
            self._synchronized = True
            return
        for p in missing:
            self._handles[p] = self._allreduce_grad_async(p)
        for p, (handle, ctx) in list(self._handles.items()):
            if handle is None:
                self._handles[p] = self._allreduce_grad_async(p)
        for p, (handle, ctx) in self._handles.items():
            if isinstance(handle, tuple) and len(handle) == 3 and handle[0] == "plain":
                _, tensor, work = handle
                if work is not None:
                    work.wait()
                output = tensor
                if self._compression is not None and work is not None:
                    output = self._compression.decompress(tensor, ctx)
            else:
                output = self._grace.receive_step(handle, ctx)
            self._allreduce_delay[p] = self.backward_passes_per_step
            if output.data_ptr() != p.grad.data_ptr():
                p.grad.set_(output.to(p.grad.dtype).view(p.grad.shape))
        self._handles.clear()
        self._synchronized = True

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
        return super(self.__class__, self).step(closure)

    def zero_grad(self, *args, **kwargs):
        if self._handles:
            raise AssertionError("optimizer.zero_grad() was called after loss.backward() but before optimizer.step() "
                                 "or optimizer.synchronize(). This is prohibited as it can cause a race condition.")
        if self._flat is not None or self._grad_accs:
            kwargs["set_to_none"] = False  # gradients are exchanged in place; keep their storage
            args = ()
        return super(self.__class__, self).zero_grad(*args, **kwargs)


def DistributedOptimizer(optimizer, grace=None, named_parameters=None, compression=None, backward_passes_per_step=1,
                         op=Average, gradient_predivide_factor=1.0, num_groups=0, flat=None, always_hook=False):
    """Wrap ``optimizer`` so that gradients are exchanged through ``grace``.

    Mirrors ``hvd.DistributedOptimizer(optimizer, grace=..., named_parameters=...)``
    of the reference (``patch_files/horovod/torch/optimizer.py:451-519``).
    ``num_groups > 0`` and ``op != Average`` bypass ``grace`` exactly as there.
    """
    if gradient_predivide_factor != 1.0 and op != Average:
        raise ValueError("gradient_predivide_factor not supported with op != Average")
    cls = type(optimizer.__class__.__name__, (optimizer.__class__,), dict(_DistributedOptimizer.__dict__))
    if flat is None:
        flat = getattr(optimizer, "flat", None)
    obj = cls.__new__(cls)
    cls.__init__(obj, optimizer.param_groups, named_parameters, grace, compression, backward_passes_per_step, op,
                 gradient_predivide_factor, num_groups, flat, always_hook)
    # keep what the wrapped optimizer had already set up (per-parameter state, flat buffers and
    # momentum of FusedSGD, ...): everything except what this wrapper itself owns
    own = {"param_groups", "defaults", "_grace", "_compression", "_parameter_names", "backward_passes_per_step",
           "_allreduce_delay", "op", "gradient_predivide_factor", "_num_groups", "_handles", "_grad_accs",
           "_requires_update", "_synchronized", "_should_synchronize", "_flat", "_bucket_events", "_side_stream"}
    for key, value in optimizer.__dict__.items():
        if key not in own and not key.startswith("_optimizer_") and not key.startswith("_zero_grad_profile"):
            obj.__dict__[key] = value
    return obj
