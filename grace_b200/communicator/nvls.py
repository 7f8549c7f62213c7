"""Uncompressed all-reduce through NVSwitch multicast, as a GRACE communicator.

``NvlsAllreduce`` serves the ``none`` compressor with no memory: the gradient is
averaged by one cooperative kernel (``csrc/dense_allreduce.cu``) in which every
rank reduces 1/W of the buffer with ``multimem.ld_reduce`` and broadcasts the
result with ``multimem.st``.  Tensors that already live in the communicator's
symmetric buffer (``buffer()``; ``FlatParams(..., grad_buffer=...)``) are reduced
in place with no staging copy; any other tensor is staged by the same kernel.

Where multicast is not available (one rank, no NVSwitch, CPU tensors) or the
compressor / memory is anything else, calls go to ``fallback`` (the peer-load
fused exchange or the library all-reduce), so the class can be constructed
unconditionally.

Reference behaviour covered: ``Allreduce`` with ``NoneCompressor``
(``grace_dl/dist/communicator/allreduce.py:6-13``, ``compressor/none.py:4-12``):
sum over ranks divided by the world size.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import distributed as dist

from ..core import Communicator


class NvlsAllreduce(Communicator):
    def __init__(self, compressor, memory, world_size: int, fallback: Communicator, group=None, device=None,
                 timeout_ms: float = 10000.0, comm_sms: Optional[int] = None, min_numel: int = 1 << 16,
                 min_world: int = 4):
        super().__init__(compressor, memory, world_size)
        self.fallback = fallback
        self.group = group
        self.device = torch.device(device) if device is not None else None
        self.timeout_ms = timeout_ms
        self.comm_sms = comm_sms
        self.min_numel = min_numel       # below this a library call or the peer-load kernel is quicker
        # a multimem load moves (1 + 1/W) N bytes per direction: slower than the peer-load exchange below 4 ranks
        # (measured at 2 ranks, 256 Mi floats: 2.79 ms in place against 2.14 ms; NCCL 2.26 ms)
        self.min_world = min_world
        self.inplace = True
        self._buf = None                 # staging buffer for tensors that live elsewhere (grown on demand)
        self._resident = []              # buffers handed out by buffer(): their tensors are reduced in place
        self._unavailable = False
        self._channel = None
        self.launches = 0

    # ------------------------------------------------------------------
    def _eligible(self, tensor: torch.Tensor) -> bool:
        from ..compressor.none import NoneCompressor
        from ..memory.none import NoneMemory

        return (tensor.is_cuda and not self._unavailable and self.world_size >= max(2, self.min_world)
                and isinstance(self.compressor, NoneCompressor) and isinstance(self.memory, NoneMemory))

    def _setup(self, device) -> bool:
        """Flags and status words on the symmetric heap (collective on first use)."""
        from ..ops.exchange import ExchangeChannel
        from ..parallel.symm import SymmetricHeap

        if self._unavailable:
            return False
        if self.device is None:
            self.device = device
        if self._channel is None:
            heap = SymmetricHeap.create(1 << 16, group=self.group, device=self.device)
            self._channel = ExchangeChannel(heap, 256, 1, self.timeout_ms, self.comm_sms)
        return True

    def _new_buffer(self, numel: int):
        from ..parallel.nvls import NvlsBuffer

        buf = NvlsBuffer.create(max(int(numel), 1 << 16), self.group, self.device)
        if buf is None:
            self._unavailable = True
        return buf

    def _find(self, t: torch.Tensor):
        for b in self._resident:
            if b.contains(t):
                return b
        return None

    def _ensure(self, t: torch.Tensor) -> bool:
        """Make sure ``t`` can be reduced: it lives in a buffer handed out by ``buffer()``, or a staging buffer of
        at least its size exists (collective on first use / growth; every rank sees the same sizes)."""
        if not self._setup(t.device):
            return False
        if self._find(t) is not None:
            return True
        if self._buf is None or self._buf.numel < t.numel():
            buf = self._new_buffer(1 << max(16, (t.numel() - 1).bit_length()))
            if buf is None:
                return False
            self._buf = buf
        return True

    def buffer(self, numel: int, device=None) -> Optional[torch.Tensor]:
        """A tensor of ``numel`` floats in symmetric memory with a multicast mapping of its own (None when
        multicast is unavailable).  Gradients kept there are reduced in place.  Collective: every rank must
        call it with the same size, in the same order."""
        if self.world_size < max(2, self.min_world) or not torch.cuda.is_available():
            return None
        device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if not self._setup(device):
            return None
        buf = self._new_buffer(numel)
        if buf is None:
            return None
        self._resident.append(buf)
        return buf.tensor[:numel]

    # ------------------------------------------------------------------
    def _allreduce(self, flat: torch.Tensor, out: torch.Tensor):
        from ..ops import native
        from ..ops.exchange import _stream_ptr

        C = native()
        ch = self._channel
        n = flat.numel()
        assert n % 4 == 0 and flat.dtype == torch.float32 and out.dtype == torch.float32
        home = self._find(flat)
        if home is not None:
            symm_ptr, mc_ptr = flat.data_ptr(), home.multicast_of(flat)
        else:
            symm_ptr, mc_ptr = self._buf.base_ptr, self._buf.multicast_ptr
        out_ptr = out.data_ptr()
        if out_ptr == flat.data_ptr() and symm_ptr == flat.data_ptr():
            out_ptr = symm_ptr                       # fully in place
        from ..utils import timeline

        tl = timeline.active()
        tok = tl.begin("dense %d" % n, "nvls.allreduce", device=True, numel=n, staged=home is None) if tl else None
        seq = ch.next_seq()
        grid = self._grid = getattr(self, "_grid", None) or C.dense_max_grid(ch.heap.device.index, ch.sm_limit)
        grid = max(1, min(grid, -(-n // (4 * 512))))
        heap = ch.heap
        scale = (1.0 / self.world_size) if self.compressor.average else 1.0
        C.dense_allreduce(flat.data_ptr(), out_ptr, symm_ptr, mc_ptr, n, scale, ch.barrier.data_ptr(),
                          ch.status.data_ptr(), ch.ready2_off, heap.rank, heap.world, seq, ch.timeout_ns, heap.bases,
                          ch.ready_off, ch.ack_off, grid, _stream_ptr())
        ch.post_status()
        self.launches += 1
        if tok is not None:
            tl.end(tok)

    def step_flat(self, flat: torch.Tensor, layout=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Average a flat fp32 buffer over the ranks (``layout`` is accepted for interface parity and ignored)."""
        usable = (self._eligible(flat) and flat.dtype == torch.float32 and flat.numel() % 4 == 0
                  and flat.data_ptr() % 16 == 0 and flat.is_contiguous() and self._ensure(flat))
        if not usable:
            if layout is not None and hasattr(self.fallback, "step_flat"):
                return self.fallback.step_flat(flat, layout, out)
            return self._library(flat, out)
        out = flat if out is None else out
        self._allreduce(flat, out)
        return out

    def _library(self, flat: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
        res = flat if out is None else out.copy_(flat)
        if self.world_size > 1:
            dist.all_reduce(res, group=self.group)
            if self.compressor.average:
                res.div_(self.world_size)
        return res

    def step(self, tensor: torch.Tensor, name: str) -> torch.Tensor:
        n = tensor.numel()
        if (not self._eligible(tensor) or n < self.min_numel or tensor.dtype != torch.float32 or n % 4
                or not tensor.is_contiguous() or tensor.data_ptr() % 16 or not self._ensure(tensor)):
            return self.fallback.step(tensor, name)
        flat = tensor.detach().reshape(-1)
        out = flat if self.inplace else torch.empty_like(flat)
        self._allreduce(flat, out)
        return out.view(tensor.shape)

    def send_step(self, tensor, name):
        out = self.step(tensor, name)
        ev = None
        if out.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
        return ("nvls", out, ev), None

    def receive_step(self, handles, ctx):
        if isinstance(handles, tuple) and len(handles) == 3 and handles[0] == "nvls":
            _, out, ev = handles
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
            return out
        return self.fallback.receive_step(handles, ctx)

    def send_receive(self, tensors, name, ctx):
        return self.fallback.send_receive(tensors, name, ctx)

    def check(self):
        """Raise ``GraceCommError`` if a bounded wait of an earlier launch ran out."""
        if self._channel is not None:
            self._channel.check()
        if hasattr(self.fallback, "check"):
            self.fallback.check()

    def reset(self):
        """After a ``GraceCommError``: clear flags and sequence numbers (call on every rank, then barrier on the host)."""
        if self._channel is not None:
            self._channel.reset()
        if hasattr(self.fallback, "reset"):
            self.fallback.reset()

    def state_dict(self):
        return self.fallback.state_dict() if hasattr(self.fallback, "state_dict") else super().state_dict()

    def load_state_dict(self, state):
        if hasattr(self.fallback, "load_state_dict"):
            self.fallback.load_state_dict(state)

    def stats(self):
        s = dict(self.fallback.stats()) if hasattr(self.fallback, "stats") else {}
        s["nvls_launches"] = self.launches
        s["nvls"] = self._buf is not None or bool(self._resident)
        return s
