"""``FusedSGD``: torch.optim.SGD semantics, one kernel launch per step.

With ``flat=FlatParams(...)`` parameters, gradients and momentum live in flat
buffers and the step is a single streaming kernel (``csrc/sgd.cu``,
``launch_fused_sgd``), which can also zero the gradient buffer for the next
backward.  Without it, a pointer table of every (param, grad, momentum) is
kept on the device and one table kernel updates the whole model
(``launch_multi_sgd``).  On CPU tensors it falls back to the plain formula.
Replaces ``torch.optim.SGD`` as used by the reference's examples
(``examples/dist/CIFAR10-dawndist/torch_backend.py:150-162``).
"""
from __future__ import annotations

import struct
from typing import Optional

import numpy as np
import torch


class FusedSGD(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, flat=None,
                 zero_grad_in_step=False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        defaults = dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov)
        super().__init__(params, defaults)
        self.flat = flat
        self.zero_grad_in_step = zero_grad_in_step
        self.grad_scale = 1.0
        self._flat_buf: Optional[torch.Tensor] = None
        self._steps = 0
        self._tables = {}

    # -- flat path ----------------------------------------------------------
    def _step_flat(self):
        from ..ops import native

        g = self.param_groups[0]
        fp = self.flat
        first = self._flat_buf is None
        if first:
            self._flat_buf = torch.zeros_like(fp.flat_p)
        native().fused_sgd(
            fp.flat_p.data_ptr(), fp.flat_g.data_ptr(), self._flat_buf.data_ptr(), fp.layout.total, float(g["lr"]),
            float(g["momentum"]), float(g["dampening"]), float(g["weight_decay"]), int(g["nesterov"]), int(first),
            int(self.zero_grad_in_step), float(self.grad_scale), torch.cuda.current_stream().cuda_stream)

    # -- pointer-table path ---------------------------------------------------
    def _step_table(self, gi, group):
        from ..ops import native

        C = native()
        params = [p for p in group["params"] if p.grad is not None]
        if not params:
            return
        first = False
        rows = []
        for p in params:
            st = self.state[p]
            if "momentum_buffer" not in st:
                st["momentum_buffer"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                st["fresh"] = True
            if not (p.is_contiguous() or p.data.is_contiguous(memory_format=torch.channels_last)):
                raise ValueError("FusedSGD needs dense parameters")
            grad = p.grad
            if grad.stride() != p.stride():
                grad = torch.empty_like(p, memory_format=torch.preserve_format).copy_(grad)
                p.grad = grad
            rows.append((p.data_ptr(), grad.data_ptr(), st["momentum_buffer"].data_ptr(), p.numel()))
        fresh = [self.state[p].pop("fresh", False) for p in params]
        first = all(fresh)
        if any(fresh) and not first:
            raise RuntimeError("FusedSGD: parameters joined the group after the first step")
        key = tuple(rows)
        cached = self._tables.get(gi)
        if cached is None or cached[0] != key:
            chunk = C.sgd_table_chunk()
            table = b"".join(struct.pack("<QQQiI", a, b, c, n, 0) for a, b, c, n in rows)
            blocks = []
            for ti, (_, _, _, n) in enumerate(rows):
                for c in range((n + chunk - 1) // chunk):
                    blocks.append((ti, c))
            dev = params[0].device
            t_dev = torch.from_numpy(np.frombuffer(table, dtype=np.uint8).copy()).to(dev)
            b_dev = torch.tensor(blocks, dtype=torch.int32, device=dev).contiguous()
            cached = (key, t_dev, b_dev, len(blocks))
            self._tables[gi] = cached
        _, t_dev, b_dev, nblocks = cached
        C.multi_sgd(t_dev.data_ptr(), b_dev.data_ptr(), nblocks, float(group["lr"]), float(group["momentum"]),
                    float(group["dampening"]), float(group["weight_decay"]), int(group["nesterov"]), int(first),
                    0, float(self.grad_scale), torch.cuda.current_stream().cuda_stream)

    def _step_cpu(self, group):
        for p in group["params"]:
            if p.grad is None:
                continue
            d = p.grad * self.grad_scale
            if group["weight_decay"] != 0:
                d = d + group["weight_decay"] * p.data
            if group["momentum"] != 0:
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = d.clone()
                else:
                    st["momentum_buffer"].mul_(group["momentum"]).add_(d, alpha=1 - group["dampening"])
                buf = st["momentum_buffer"]
                d = d + group["momentum"] * buf if group["nesterov"] else buf
            p.data.add_(d, alpha=-group["lr"])

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.flat is not None and self.flat.flat_p.is_cuda:
            self._step_flat()
        else:
            for gi, group in enumerate(self.param_groups):
                ps = [p for p in group["params"] if p.grad is not None]
                if ps and ps[0].is_cuda:
                    self._step_table(gi, group)
                else:
                    self._step_cpu(group)
        self._steps += 1
        return loss

    # -- checkpoint: the flat momentum buffer is exported in torch.optim.SGD's format -------------
    def _flat_slices(self, flat_tensor):
        fp = self.flat
        by_id = {id(p): (off, p) for p, off in zip(fp.params, fp.layout.offsets)}
        out = []
        for group in self.param_groups:
            for p in group["params"]:
                off, _ = by_id.get(id(p), (None, None))
                out.append(None if off is None else flat_tensor[off : off + p.numel()])
        return out

    def state_dict(self):
        sd = super().state_dict()
        if self.flat is not None and self._flat_buf is not None:
            from ..parallel.flat import _dense_view

            idx = 0
            for group in self.param_groups:
                for p in group["params"]:
                    off = dict((id(q), o) for q, o in zip(self.flat.params, self.flat.layout.offsets)).get(id(p))
                    if off is not None:
                        sd["state"].setdefault(idx, {})["momentum_buffer"] = _dense_view(
                            self._flat_buf, off, p.data).clone()
                    idx += 1
        return sd

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        if self.flat is None:
            return
        from ..parallel.flat import _dense_view

        found = False
        buf = torch.zeros_like(self.flat.flat_p)
        for p, off in zip(self.flat.params, self.flat.layout.offsets):
            st = self.state.get(p, {})
            if "momentum_buffer" in st and st["momentum_buffer"] is not None:
                _dense_view(buf, off, p.data).copy_(st.pop("momentum_buffer"))
                found = True
        if found:
            self._flat_buf = buf

    def zero_grad(self, set_to_none: bool = False):
        if self.flat is not None:
            if not self.zero_grad_in_step:
                self.flat.zero_grad()
            return
        super().zero_grad(set_to_none=set_to_none)
