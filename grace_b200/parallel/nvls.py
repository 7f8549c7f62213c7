"""Symmetric buffers with an NVSwitch multicast address.

``NvlsBuffer`` is one fp32 buffer that every rank of a process group holds a
copy of, mapped twice: at its ordinary local address, and at a *multicast*
address through which one ``multimem.ld_reduce`` returns the sum of all W
copies (added inside the switch) and one ``multimem.st`` writes all W copies.
The allocation, the exchange of the memory handles and the binding to the
multicast object are done by ``torch.distributed._symmetric_memory``; the
kernels that use the two addresses are this package's own
(``csrc/dense_allreduce.cu``).

Multicast needs NVSwitch-connected GPUs and at least two ranks;
``NvlsBuffer.create`` returns ``None`` where it is not available, and callers
fall back to the peer-load kernels.

A rank must not die while its memory is bound to a multicast object (the other
GPUs then see NVLink faults), so failure-handling tests and elastic runs keep
this path off; it is opt-in (``grace_from_params({..., "nvls": True})``).

The reference has no counterpart: its uncompressed path is one library
all-reduce per tensor (``grace_dl/dist/communicator/allreduce.py:6-13``).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import distributed as dist


class NvlsBuffer:
    last_error = None   # why the last create() on this rank found no multicast (for diagnostics)

    def __init__(self, tensor: torch.Tensor, handle, multicast_ptr: int):
        self.tensor = tensor
        self.handle = handle          # keeps the mappings alive
        self.multicast_ptr = multicast_ptr
        self.numel = tensor.numel()

    @property
    def base_ptr(self) -> int:
        return self.tensor.data_ptr()

    def contains(self, t: torch.Tensor) -> bool:
        p = t.data_ptr()
        return self.base_ptr <= p and p + t.numel() * t.element_size() <= self.base_ptr + 4 * self.numel

    def multicast_of(self, t: torch.Tensor) -> int:
        """Multicast address of a tensor that lives inside this buffer."""
        return self.multicast_ptr + (t.data_ptr() - self.base_ptr)

    @classmethod
    def create(cls, numel: int, group=None, device=None) -> Optional["NvlsBuffer"]:
        if not (dist.is_available() and dist.is_initialized() and torch.cuda.is_available()):
            return None
        group = group if group is not None else dist.group.WORLD
        if dist.get_world_size(group) < 2:
            return None
        device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        t = handle = None
        mc = 0
        try:
            import torch.distributed._symmetric_memory as symm_mem

            t = symm_mem.empty(int(numel), dtype=torch.float32, device=device)
            try:
                handle = symm_mem.rendezvous(t, group)
            except TypeError:
                handle = symm_mem.rendezvous(t, group.group_name)
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)
        except (ImportError, RuntimeError, AttributeError, NotImplementedError) as e:
            cls.last_error = "%s: %s" % (type(e).__name__, str(e).splitlines()[0] if str(e) else "")
            mc = 0
        # every rank must take the same branch: agree on the outcome
        flag = torch.tensor([1 if mc else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            return None
        t.zero_()
        return cls(t, handle, mc)
