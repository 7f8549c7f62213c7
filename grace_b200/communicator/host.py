"""``HostExchange``: the fused exchange protocol among CPU ranks.

The GPU kernels of this package publish encoded gradients in send slots of a
symmetric heap, signal them with sequence-numbered flags, read the peers'
slots directly, acknowledge what they read, and give every wait a deadline
that ends in a status block instead of a hang.  ``csrc/host_exchange.cpp``
runs the same state machine on the host: every rank owns a POSIX
shared-memory segment that all ranks of the machine map, and
``compensate -> encode -> publish -> pull + decode-sum -> acknowledge`` is one
native call per tensor (no Gloo collective, no W dense decompress passes).

It serves two purposes: CPU tensors get a fused path behind the same
communicator API (``grace_from_params({..., 'fused': True, 'host_protocol':
True})``), and the protocol itself - slot reuse, a late peer, a peer that never
publishes, agreement and recovery - runs among really concurrent ranks
(processes of a ``torch.distributed`` group, or threads of one process through
``ThreadWorld``) on a machine without a GPU.

Pairs covered: TopK / Threshold / RandomK with none or residual memory, TopK / DGC with
the momentum-corrected DGC memory (exact k-th magnitude, optional gradient
clipping by the ranks' sums of squares), QSGD
(any bucket size, up to 32767 levels), TernGrad, natural compression (the
CUDA extension's code table; stochastic or deterministic), 8-bit, 1-bit and
fp16 with none or residual memory, signSGD / signum, EF-signSGD with its
memory, PowerSGD (ranks up to 16, with or without its error-feedback memory;
1-D tensors travel uncompressed) and no compression.  Stochastic codecs draw the Philox stream of the
GPU path.  Anything else uses the library ``Allgather`` path.

The reference's CPU ranks meet only inside Gloo collectives
(``grace_dl/dist/communicator/allgather.py:8-45``).
"""
from __future__ import annotations

import ctypes
import threading
import uuid
from typing import Dict, List, Optional

import numpy as np
import torch
from torch import distributed as dist

from .. import compressor as C_
from .. import memory as M_
from ..compressor._common import topk_count
from ..core import Communicator
from .allgather import Allgather

PHASE_COMPRESS, PHASE_PUBLISH, PHASE_EXCHANGE, PHASE_ALL = 1, 2, 4, 7
TOPK, THRESHOLD, QSGD, SIGN, EFSIGN, DENSE, TERNGRAD, NATURAL, U8BIT, ONEBIT, FP16, RANDOMK, QSGDX, LOWRANK = range(14)
_ALIGN = 64


# ----------------------------------------------------------------------------- how the ranks meet
class DistWorld:
    """Ranks are the processes of a ``torch.distributed`` group (gloo on CPU)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        box = [uuid.uuid4().hex[:12] if self.rank == 0 else None]
        if self.world > 1:
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self.token = box[0]
        self._serial = 0

    def next_serial(self) -> int:
        """Number of the next heap these ranks create together (part of its shared-memory name)."""
        self._serial += 1
        return self._serial

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)


class ThreadWorld:
    """W ranks as threads of ONE process (the native call releases the interpreter lock, so the ranks really run
    side by side and really wait for each other).  ``view(r)`` is what rank ``r`` hands to ``HostExchange``."""

    def __init__(self, world: int):
        self.world = int(world)
        self.token = uuid.uuid4().hex[:12]
        self._barrier = threading.Barrier(self.world)
        self._serials = [0] * self.world   # heaps created so far, per rank (all ranks create them in the same order)

    def view(self, rank: int) -> "_ThreadRank":
        return _ThreadRank(self, rank)

    def run(self, fn, timeout_s: float = 60.0) -> List:
        """``fn(rank_view)`` on every rank; returns the results in rank order, re-raises the first exception."""
        results: List = [None] * self.world
        errors: List = [None] * self.world

        def body(r):
            try:
                results[r] = fn(self.view(r))
            except BaseException as e:   # noqa: BLE001 - reported to the caller below
                errors[r] = e
                self._barrier.abort()

        threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout_s)
        for e in errors:
            if e is not None and not isinstance(e, threading.BrokenBarrierError):
                raise e
        for e in errors:
            if e is not None:
                raise e
        if any(t.is_alive() for t in threads):
            raise TimeoutError("a rank thread did not finish within %.0f s" % timeout_s)
        return results


class _ThreadRank:
    def __init__(self, owner: ThreadWorld, rank: int):
        self.owner, self.rank, self.world, self.token = owner, rank, owner.world, owner.token

    def next_serial(self) -> int:
        self.owner._serials[self.rank] += 1
        return self.owner._serials[self.rank]

    def barrier(self):
        self.owner._barrier.wait(timeout=60.0)


# ----------------------------------------------------------------------------- shared memory
class HostHeap:
    """One shared-memory segment per rank, each mapped by every rank; offsets come from a bump allocator that all
    ranks drive with the same requests.  The names are unlinked as soon as everybody has mapped them, so nothing
    stays behind in ``/dev/shm`` when a rank dies."""

    def __init__(self, nbytes: int, world):
        from ..ops import native

        self._C = native()
        self.nbytes = (int(nbytes) + 4095) // 4096 * 4096
        self.rank, self.world = world.rank, world.world
        serial = world.next_serial()   # the same number on every rank: heaps are created in the same order

        def name(r):
            return "/grace_%s_%d_%d" % (world.token, serial, r)

        self.bases: List[int] = [0] * self.world
        self._cursor = 0
        self._closed = False
        self.bases[self.rank] = self._C.host_heap_create(name(self.rank), self.nbytes)
        try:
            world.barrier()
            for r in range(self.world):
                if r != self.rank:
                    self.bases[r] = self._C.host_heap_open(name(r), self.nbytes)
            world.barrier()
        finally:
            # also when a peer never showed up: the name must not outlive this call (the mappings keep the memory)
            self._C.host_heap_unlink(name(self.rank))

    def alloc(self, nbytes: int) -> int:
        off = (self._cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        if off + nbytes > self.nbytes:
            raise MemoryError("host heap exhausted: need %d bytes at offset %d of %d" % (nbytes, off, self.nbytes))
        self._cursor = off + nbytes
        return off

    def view(self, offset: int, numel: int, dtype=np.uint64, rank: Optional[int] = None) -> np.ndarray:
        r = self.rank if rank is None else rank
        nbytes = numel * np.dtype(dtype).itemsize
        buf = (ctypes.c_char * nbytes).from_address(self.bases[r] + offset)
        return np.frombuffer(buf, dtype=dtype, count=numel)

    def close(self):
        if not self._closed:
            self._closed = True
            for b in self.bases:
                if b:
                    self._C.host_heap_close(b, self.nbytes)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _HostPlan:
    """Flags, status block and two send slots of one tensor, plus its error-feedback state."""

    def __init__(self, owner: "HostExchange", name: str, numel: int, codec: Optional[int] = None, shape=None):
        C = owner._C
        self.name, self.numel = name, numel
        comp = owner.compressor
        self.codec = codec = owner._codec if codec is None else codec
        self.k = 0
        if codec == LOWRANK:
            self._init_lowrank(owner, shape)
            return
        if codec in (TOPK, RANDOMK):
            self.k = topk_count(numel, comp.compress_ratio)
        elif codec == THRESHOLD:
            self.k = max(1, int(numel * owner.max_ratio))
        self.bucket = int(getattr(comp, "bucket_size", 0)) if codec == QSGDX else 0
        self.two_phase = owner.mode == "alltoall" and codec in (QSGD, NATURAL, FP16, DENSE)
        if self.two_phase:
            self.slot_bytes = C.host_two_phase_slot_bytes(codec, numel, owner.world_size)
        else:
            self.slot_bytes = C.host_slot_bytes(codec, numel, self.bucket if codec == QSGDX else self.k)
        self.clip = codec == TOPK and owner._needs_u and bool(getattr(owner.memory, "gradient_clipping", False))
        self._carve(owner, flag_pads=3 if (self.two_phase or self.clip) else 2)   # the third pad serves either use
        # the key of the random stream: as the GPU path derives it for a single tensor (name and padded length)
        self.seed = _name_seed(owner.seed, name + str((numel + 127) // 128 * 128))
        if codec == RANDOMK:   # the positions are keyed by the tensor's name alone, as on the GPU
            self.seed = _name_seed(owner.seed, name)
        self.seq = 0          # sequence number of the last exchange started
        self.steps = 0
        plain_dense = codec == DENSE and owner._codec == LOWRANK   # a 1-D tensor next to PowerSGD matrices
        self.acc = torch.zeros(numel, dtype=torch.float32) if (owner._needs_acc and not plain_dense) else None
        self.mom = torch.zeros(numel, dtype=torch.float32) if owner._needs_mom else None
        self.u = torch.zeros(numel, dtype=torch.float32) if owner._needs_u else None

    def _carve(self, owner, flag_pads: int):
        """Flag pads (ready, ack and, for the low-rank exchange, the second rendezvous), status block, two slots."""
        C = owner._C
        need = flag_pads * C.HOST_MAX_WORLD * 8 + 64 + 2 * self.slot_bytes + 8 * _ALIGN
        heap = self.heap = owner._heap_with_room(need)
        self.flag_words = flag_pads * C.HOST_MAX_WORLD
        self.ready_off = heap.alloc(self.flag_words * 8)   # ready[MAX_WORLD], ack[MAX_WORLD] (, ready2[MAX_WORLD])
        self.ack_off = self.ready_off + C.HOST_MAX_WORLD * 8
        self.ready2_off = self.ready_off + 2 * C.HOST_MAX_WORLD * 8 if flag_pads > 2 else 0
        self.status_off = heap.alloc(64)
        self.slot_off = [heap.alloc(self.slot_bytes), heap.alloc(self.slot_bytes)]

    def _init_lowrank(self, owner, shape):
        """PowerSGD on one matrix: rows = shape[0], columns = the rest; Q starts from the orthogonalised N(0, 1)
        draw the GPU path uses (same seed: identical on every rank)."""
        import zlib

        from ..ops.lowrank import orthogonal_init

        self.rows = int(shape[0])
        self.cols = self.numel // self.rows
        self.rank = min(self.rows, self.cols, int(owner.compressor.rank))
        self.slot_bytes = owner._C.host_lowrank_slot_bytes(self.rows, self.cols, self.rank)
        self._carve(owner, flag_pads=3)
        self.seed = 0
        self.seq = self.steps = 0
        self.bucket = 0
        self.two_phase = self.clip = False
        self.acc = torch.zeros(self.numel, dtype=torch.float32) if isinstance(owner.memory, M_.PowerSGDMemory) else None
        self.mom = self.u = None
        self.q = orthogonal_init(self.cols, self.rank, owner.seed ^ zlib.crc32(self.name.encode("utf8")),
                                 "cpu").contiguous()
        self.p_work = torch.zeros(self.rows * self.rank, dtype=torch.float32)

    def status(self) -> np.ndarray:
        return self.heap.view(self.status_off, 8, np.uint32)

    def reset(self):
        self.heap.view(self.ready_off, self.flag_words, np.uint64)[:] = 0
        self.status()[:] = 0
        self.seq = 0


class HostExchange(Communicator):
    def __init__(self, compressor, memory, world_size, world=None, group=None, seed=0, timeout_ms=10000.0,
                 arena_mb=16, max_ratio=0.25, store=None, rank=None, mode="allgather"):
        """``world``: how the ranks meet (``DistWorld`` by default: the processes of ``group``; a
        ``ThreadWorld.view(r)`` for ranks that are threads).  ``timeout_ms``: limit of every wait for a peer.
        ``store``: a ``torch.distributed`` store for ``agree`` / ``recover`` (process ranks only).  ``mode``:
        ``"alltoall"`` selects the two-phase exchange (compressed reduce-scatter, re-encode, compressed all-gather:
        the reference's ``AllToAll`` communicator) for QSGD with 128-element buckets, natural compression, fp16 and
        no compression; every other codec keeps the all-gather form."""
        super().__init__(compressor, memory, world_size)
        self.mode = mode
        from ..ops import native
        from ..utils.faults import FaultPlan

        self._C = native()
        self._world = world
        self.group = group
        self.seed = int(seed)
        self.timeout_ms = float(timeout_ms)
        self.arena_bytes = int(arena_mb * (1 << 20))
        self.max_ratio = float(max_ratio)
        self.store = store
        self._rank = rank
        self._epoch = 0
        self._heaps: List[HostHeap] = []
        self._plans: Dict[tuple, _HostPlan] = {}
        self._fallback = Allgather(compressor, memory, world_size)
        self._faults = FaultPlan.from_env()
        self._pending_state = None
        self._resolve()

    # ------------------------------------------------------------------
    def _resolve(self):
        comp, mem = self.compressor, self.memory
        self._codec = None
        self._needs_acc = isinstance(mem, (M_.ResidualMemory, M_.EFSignSGDMemory, M_.DgcMemory))
        self._needs_u = isinstance(mem, M_.DgcMemory)
        self._needs_mom = isinstance(comp, C_.SignumCompressor)
        plain = isinstance(mem, (M_.NoneMemory, M_.ResidualMemory))
        if isinstance(comp, C_.PowerSGDCompressor):
            if isinstance(mem, (M_.PowerSGDMemory, M_.NoneMemory)) and 1 <= int(comp.rank) <= 16:
                self._codec = LOWRANK
                self._needs_acc = False   # the low-rank plans own their residual; 1-D tensors travel uncompressed
        elif isinstance(mem, M_.DgcMemory):
            if isinstance(comp, (C_.TopKCompressor, C_.DgcCompressor)):
                self._codec = TOPK   # with gradient_clipping: sums of squares are exchanged before the encode
        elif isinstance(comp, (C_.TopKCompressor, C_.DgcCompressor)) and plain:
            self._codec = TOPK
        elif isinstance(comp, C_.ThresholdCompressor) and plain:
            self._codec = THRESHOLD
        elif isinstance(comp, C_.RandomKCompressor) and plain:
            self._codec = RANDOMK
        elif isinstance(comp, C_.QSGDCompressor) and plain and comp.bucket_size == 128 and comp.quantum_num < 128:
            self._codec = QSGD
        elif isinstance(comp, C_.QSGDCompressor) and plain and comp.bucket_size >= 1 and comp.quantum_num < 32768:
            self._codec = QSGDX   # any bucket size, int16 codes
        elif isinstance(comp, (C_.SignSGDCompressor, C_.SignumCompressor)) and plain:
            self._codec = SIGN
        elif isinstance(comp, C_.EFSignSGDCompressor) and isinstance(mem, (M_.EFSignSGDMemory, M_.NoneMemory)):
            self._codec = EFSIGN
        elif isinstance(comp, C_.NoneCompressor) and isinstance(mem, M_.NoneMemory):
            self._codec = DENSE
        elif plain:
            for cls, codec in ((C_.TernGradCompressor, TERNGRAD), (C_.NaturalCompressor, NATURAL),
                               (C_.U8bitCompressor, U8BIT), (C_.OneBitCompressor, ONEBIT), (C_.FP16Compressor, FP16)):
                if isinstance(comp, cls):
                    self._codec = codec
                    break

    def supported(self, tensor: torch.Tensor) -> bool:
        return (self._codec is not None and not tensor.is_cuda and tensor.is_floating_point()
                and 0 < tensor.numel() < 2 ** 31)

    def _meet(self):
        if self._world is None:
            self._world = DistWorld(self.group)
        if self._world.world != self.world_size:
            raise ValueError("world_size=%d but the ranks that meet are %d" % (self.world_size, self._world.world))
        return self._world

    def _heap_with_room(self, nbytes: int) -> HostHeap:
        """The newest heap if ``nbytes`` still fit, else a new one: a collective step, so plans must be created
        in the same order on every rank (``prepare``)."""
        world = self._meet()
        if self._heaps and self._heaps[-1].nbytes - self._heaps[-1]._cursor >= nbytes + _ALIGN:
            return self._heaps[-1]
        heap = HostHeap(max(self.arena_bytes, nbytes + 4096), world)
        self._heaps.append(heap)
        return heap

    def prepare(self, named_tensors):
        """Create the plans now, in name order (heap creation is collective; gradient hooks may fire in any order)."""
        for name, t in sorted(((n, t) for n, t in named_tensors), key=lambda kv: kv[0]):
            if self.supported(t):
                self._plan(name, t.numel(), tuple(t.shape))

    def _plan(self, name: str, numel: int, shape=None) -> _HostPlan:
        key = (name, numel)
        plan = self._plans.get(key)
        if plan is None:
            codec = None
            if self._codec == LOWRANK:   # matrices are compressed, 1-D tensors are exchanged as they are
                matrix = shape is not None and len(shape) >= 2 and int(shape[0]) >= 1 and numel // int(shape[0]) >= 1
                codec = LOWRANK if matrix else DENSE
            plan = self._plans[key] = _HostPlan(self, name, numel, codec, shape)
            if self._pending_state:
                self._restore_plan(plan, self._pending_state)
        return plan

    # ------------------------------------------------------------------
    def _coeffs(self, plan: _HostPlan):
        mem, first = self.memory, plan.steps == 0
        if isinstance(mem, M_.ResidualMemory):
            return (0.0, 1.0) if first else (float(mem.beta), float(mem.gamma))
        if isinstance(mem, M_.EFSignSGDMemory):
            return (0.0, 1.0) if first else (1.0, float(mem.learning_rate))
        return 0.0, 1.0

    def _run(self, plan: _HostPlan, g: torch.Tensor, out: torch.Tensor, phases: int):
        from ..ops.exchange import GraceCommError

        comp = self.compressor
        world = self._meet()
        if self._faults.action and (phases & PHASE_PUBLISH) and self._faults.hits("skip_publish", world.rank,
                                                                                  plan.steps):
            phases &= ~PHASE_PUBLISH   # host-side fault injection: this rank "forgets" to publish
        beta, gamma = self._coeffs(plan)
        heap = plan.heap
        if plan.codec == LOWRANK:
            rc = self._C.host_lowrank_exchange(
                world.rank, world.world, heap.bases, plan.ready_off, plan.ack_off, plan.status_off, plan.slot_off[0],
                plan.slot_off[1], plan.slot_bytes, int(self.timeout_ms * 1e6), plan.ready2_off, phases, plan.seq,
                g.data_ptr(), plan.acc.data_ptr() if plan.acc is not None else 0, out.data_ptr(), plan.q.data_ptr(),
                plan.p_work.data_ptr(), plan.rows, plan.cols, plan.rank)
            if rc != 0:
                st = plan.status()
                raise GraceCommError(int(rc), int(st[1]), int(st[2]), world.rank)
            return
        rc = self._C.host_exchange(
            world.rank, world.world, heap.bases, plan.ready_off, plan.ack_off, plan.status_off, plan.slot_off[0],
            plan.slot_off[1], plan.slot_bytes, int(self.timeout_ms * 1e6), plan.codec, phases, plan.seq,
            g.data_ptr(), plan.acc.data_ptr() if plan.acc is not None else 0,
            plan.mom.data_ptr() if plan.mom is not None else 0, out.data_ptr(), plan.numel, plan.k, beta, gamma,
            (1.0 / self.world_size) if comp.average else 1.0, float(getattr(comp, "threshold", 0.0)),
            int(bool(getattr(comp, "strict", False))), float(getattr(comp, "learning_rate", 1.0)),
            float(getattr(comp, "momentum", 0.0)), int(plan.steps == 0), int(getattr(comp, "quantum_num", 0)),
            plan.seed, plan.steps, plan.u.data_ptr() if plan.u is not None else 0,
            float(getattr(self.memory, "momentum", 0.0)), int(bool(getattr(comp, "deterministic", False))),
            plan.bucket, plan.ready2_off if plan.two_phase else 0, plan.ready2_off if plan.clip else 0)
        if rc != 0:
            st = plan.status()
            raise GraceCommError(int(rc), int(st[1]), int(st[2]), world.rank)

    def _payload_bytes(self, plan: _HostPlan) -> int:
        if plan.codec == LOWRANK:
            return 4 * (plan.rows + plan.cols) * plan.rank
        if plan.codec == RANDOMK:
            return 4 * plan.k
        return 8 * plan.k if plan.codec in (TOPK, THRESHOLD) else int(plan.slot_bytes)

    def step(self, tensor: torch.Tensor, name: str) -> torch.Tensor:
        handles, ctx = self.send_step(tensor, name)
        return self.receive_step(handles, ctx)

    # split-phase (grace_dl/torch/__init__.py:50-58): send = compensate, encode, publish; receive = pull, decode, ack
    def send_step(self, tensor: torch.Tensor, name: str):
        if not self.supported(tensor):
            return self._fallback.send_step(tensor, name)
        g = tensor.detach().reshape(-1).to(torch.float32).contiguous()
        plan = self._plan(name, g.numel(), tuple(tensor.shape))
        plan.seq += 1
        self._stats["steps"] += 1
        self._stats["dense_bytes"] += 4 * plan.numel
        self._stats["payload_bytes"] += self._payload_bytes(plan)
        out = torch.empty_like(g)
        self._run(plan, g, out, PHASE_COMPRESS | PHASE_PUBLISH)
        return ("host", plan, g, out, tensor.shape, tensor.dtype), None

    def receive_step(self, handles, ctx) -> torch.Tensor:
        if not (isinstance(handles, tuple) and handles and handles[0] == "host"):
            return self._fallback.receive_step(handles, ctx)
        _, plan, g, out, shape, dtype = handles
        self._run(plan, g, out, PHASE_EXCHANGE)
        plan.steps += 1
        return out.view(shape).to(dtype)

    def send_receive(self, tensors, name, ctx):
        return self._fallback.send_receive(tensors, name, ctx)

    def step_flat(self, flat: torch.Tensor, layout, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A whole flat buffer of named gradients (``FlatLayout``: names, offsets, numels), tensor by tensor: every
        tensor is published before the first one is pulled, so the ranks' encode passes overlap.  In place unless
        ``out`` is given.  (The call shape of ``FusedExchange.step_flat``; used by ``DistributedOptimizer`` with
        ``FlatParams`` on CPU.)"""
        out = flat if out is None else out
        pending = []
        for name, off, numel in zip(layout.names, layout.offsets, layout.numels):
            pending.append((off, numel, self.send_step(flat[off:off + numel], name)))
        for off, numel, (handles, ctx) in pending:
            out[off:off + numel] = self.receive_step(handles, ctx)
        return out

    def prepare_layouts(self, layouts, device=None):
        """Create the plans of whole buckets up front, in the order given (same on every rank)."""
        for layout in layouts:
            for name, numel in zip(layout.names, layout.numels):
                self._plan(name, numel)

    # ------------------------------------------------------------------ failures
    def check(self):
        from ..ops.exchange import GraceCommError

        for plan in self._plans.values():
            st = plan.status()
            if st[0] != 0:
                raise GraceCommError(int(st[0]), int(st[1]), int(st[2]), self._meet().rank)

    def reset(self):
        """Clear this rank's flags, status words and sequence numbers; error-feedback state is kept.  Every rank
        calls it, with a meeting of the ranks before (nobody still writes a peer's flags) and after."""
        for plan in self._plans.values():
            plan.reset()

    def agree(self, local_error: Optional[BaseException] = None, timeout_s: float = 30.0):
        """Step-boundary vote through the store: the ranks that saw a failure, the same list on every rank."""
        if self.store is None:
            raise RuntimeError("agree() needs a store (HostExchange(..., store=...))")
        failed = local_error is not None
        if not failed:
            try:
                self.check()
            except RuntimeError as e:
                local_error, failed = e, True
        return self._board().vote(self._epoch, failed, timeout_s=timeout_s,
                                  info=str(local_error)[:200] if failed else "")

    def recover(self, timeout_s: float = 30.0):
        """On every rank after a failed exchange: meet, clear the pads, meet again; the next exchange starts from
        sequence 1 with the error-feedback state intact."""
        def meet(tag):
            if self.world_size == 1:
                return
            if self.store is not None:
                self._board().barrier(self._epoch, timeout_s=timeout_s, tag=tag)
            else:
                self._meet().barrier()

        meet("quiet")
        self.reset()
        meet("clean")
        self._epoch += 1

    def _board(self):
        from ..utils.faults import ErrorBoard

        if getattr(self, "_error_board", None) is None:
            self._error_board = ErrorBoard(self.store, self._meet().rank if self._rank is None else int(self._rank),
                                           self.world_size, prefix="grace/host_error")
        return self._error_board

    def close(self):
        if self._world is not None and self._heaps and self.world_size > 1:
            self._world.barrier()
        self._plans.clear()
        for h in self._heaps:
            h.close()
        self._heaps = []

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        if not self._plans:
            return self._fallback.state_dict()
        residuals = {p.name: p.acc.clone() for p in self._plans.values() if p.acc is not None and p.u is None}
        gradients = {p.name: p.acc.clone() for p in self._plans.values() if p.u is not None}   # DGC: v
        residuals.update({p.name: p.u.clone() for p in self._plans.values() if p.u is not None})   # DGC: u
        comp = self.compressor.state_dict()
        momentums = {p.name: p.mom.clone() for p in self._plans.values() if p.mom is not None}
        if momentums:
            comp["momentums"] = momentums
        q_memory = {p.name: p.q.clone() for p in self._plans.values() if p.codec == LOWRANK}
        if q_memory:
            comp["q_memory"] = q_memory   # [columns x rank], the reference's shape
        mem = {"residuals": residuals}
        if gradients:
            mem["gradients"] = gradients
        return {"compressor": comp, "memory": mem, "world_size": self.world_size,
                "host_steps": {p.name: p.steps for p in self._plans.values()}}

    def load_state_dict(self, state):
        self._pending_state = state
        self._fallback.load_state_dict(state)
        for plan in self._plans.values():
            self._restore_plan(plan, state)

    def _restore_plan(self, plan: _HostPlan, state):
        mem = state.get("memory", {})
        res = mem.get("gradients" if plan.u is not None else "residuals", {})
        if plan.acc is not None and plan.name in res:
            plan.acc.copy_(res[plan.name].reshape(-1).to(torch.float32))
            plan.steps = max(plan.steps, 1)
        if plan.u is not None and plan.name in mem.get("residuals", {}):
            plan.u.copy_(mem["residuals"][plan.name].reshape(-1).to(torch.float32))
        moms = state.get("compressor", {}).get("momentums", {})
        if plan.mom is not None and plan.name in moms:
            plan.mom.copy_(moms[plan.name].reshape(-1).to(torch.float32))
            plan.steps = max(plan.steps, 1)
        qs = state.get("compressor", {}).get("q_memory", {})
        if plan.codec == LOWRANK and plan.name in qs and tuple(qs[plan.name].shape) == (plan.cols, plan.rank):
            plan.q.copy_(qs[plan.name].to(torch.float32))
        plan.steps = max(plan.steps, int(state.get("host_steps", {}).get(plan.name, 0)))


def _name_seed(seed: int, name: str) -> int:
    import zlib

    return ((seed & 0xFFFFFFFF) << 32) | (zlib.crc32(name.encode("utf8")) & 0xFFFFFFFF)
