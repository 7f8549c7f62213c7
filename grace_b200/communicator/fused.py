"""``FusedExchange``: one sm_100a kernel launch per gradient exchange.

Where the library communicators (``Allgather`` and friends) run
compensate -> compress -> memory.update -> collective -> W x decompress ->
aggregate as a chain of framework ops and NCCL calls, this communicator hands
the gradient, the error-feedback arenas and the peers' heap pointers to one
cooperative kernel (``csrc/sparse_exchange.cu`` or ``csrc/quant_exchange.cu``)
that does all of it, reading the other ranks' send slots over NVLink from
inside the kernel.

Supported pairs (anything else transparently uses the library ``Allgather``
path, as does every call on CPU tensors):

==================  =====================================  ==================
compressor          memory                                 kernel
==================  =====================================  ==================
TopK, DGC           none / residual / dgc                  sparse (radix select)
Threshold           none / residual                        sparse (threshold)
QSGD (any bucket    none / residual                        quantised
that is a multiple
of 4, q < 32768),
TernGrad, natural,
8-bit, fp16, none
signSGD, signum     none / residual                        quantised, vote
EF-signSGD          efsignsgd                              quantised
1-bit               none / residual                        quantised
PowerSGD            powersgd                               low-rank (tcgen05)
==================  =====================================  ==================

Threshold compression has a data-dependent payload: the send slot holds at most
``max_ratio`` (default 0.25) of the elements; what does not fit stays in the
residual (counted by ``channel.dropped()``).

Two granularities: ``step(tensor, name)`` (one tensor, API of the reference)
and ``step_flat(flat, layout)`` (a whole bucket of named tensors in one launch,
used by the DDP hook and ``DistributedOptimizer``).
"""
from __future__ import annotations

import os
import zlib
from typing import Dict, List, Optional, Sequence

import torch
from torch import distributed as dist

from ..core import Communicator
from .. import compressor as C_
from .. import memory as M_
from ..compressor._common import topk_count
from .allgather import Allgather


def _name_seed(seed: int, name: str) -> int:
    return ((seed & 0xFFFFFFFF) << 32) | (zlib.crc32(name.encode("utf8")) & 0xFFFFFFFF)


class _Arena:
    """The symmetric memory of one communicator: a few large heaps, carved up by the plans.

    A heap costs one ``cudaMalloc``, one exchange of IPC handles among the ranks and ``W - 1`` mappings; a plan
    only needs a range of it.  The first plan creates a heap of at least ``default_bytes``; a later plan that
    does not fit makes the arena grow by another heap (again a collective step, so plans must be created in the
    same order on every rank: ``FusedExchange.prepare`` does that up front, in name order)."""

    def __init__(self, create, default_bytes: int):
        self._create = create
        self.default_bytes = int(default_bytes)
        self.segments = []

    def carve(self, nbytes: int):
        if self.segments:
            try:
                return self.segments[-1].carve(nbytes)
            except MemoryError:
                pass
        need = (int(nbytes) + 255) // 256 * 256 + 256
        seg = self._create(max(self.default_bytes, need))
        self.segments.append(seg)
        return seg.carve(nbytes)

    def close(self):
        for seg in self.segments:
            seg.close()
        self.segments = []


class _VirtualSegment:
    """One arena heap of a ``VirtualWorld``: W heaps in this process, carved in lock step."""

    def __init__(self, heaps):
        self.heaps = heaps

    def carve(self, nbytes: int):
        return [h.carve(nbytes) for h in self.heaps]

    def close(self):
        for h in self.heaps:
            h.close()


class _Plan:
    """Everything one layout needs: heap, channel, segment table, arenas."""

    def __init__(self, owner: "FusedExchange", layout, kind: str):
        from ..ops import exchange as X, native

        Cn = native()
        self.layout = layout
        self.kind = kind
        self.steps = 0
        comp = owner.compressor
        device = owner.device
        nseg = len(layout.names)
        self.ks = None
        if kind == "sparse":
            self.kprefix = self.seg_seed = None
            if isinstance(comp, C_.RandomKCompressor):
                self.mode = X.SPARSE_RANDOMK
                self.ks = [topk_count(n, comp.compress_ratio) for n in layout.numels]
                self.cap = X.sparse_capacity(layout, self.ks, self.mode)
                prefix = [0]
                for k in self.ks:
                    prefix.append(prefix[-1] + k)
                self.kprefix = torch.tensor(prefix, dtype=torch.int32, device=device)
                seeds = [_name_seed(owner.seed, n) for n in layout.names]
                self.seg_seed = torch.tensor([s - (1 << 64) if s >= (1 << 63) else s for s in seeds],
                                             dtype=torch.int64, device=device)
            elif isinstance(comp, C_.ThresholdCompressor):
                self.mode = X.SPARSE_THRESHOLD
                self.cap = X.sparse_capacity(layout, [], self.mode, owner.max_ratio)
            else:
                self.mode = X.SPARSE_TOPK
                self.ks = [topk_count(n, comp.compress_ratio) for n in layout.numels]
                self.cap = X.sparse_capacity(layout, self.ks, self.mode)
            # tile-ordered lists (sender sorts by output tile, receivers build dense tiles): same decision on every rank
            self.tile = X.tile_decode_wanted(layout.total, self.cap, owner.world_size, self.mode)
            slot_bytes = Cn.sparse_slot_bytes(self.cap, layout.total if self.tile else 0)
        else:
            self.codec = owner._codec
            self.alltoall = owner.mode == "alltoall" and self.codec in (X.CODEC["qsgd"], X.CODEC["natural"],
                                                                        X.CODEC["fp16"], X.CODEC["fp32"])
            self.qsgd_bucket = self.qsgd_nbuckets = 0
            if self.codec == X.CODEC["qsgdx"]:
                # Segment.k carries the index of each tensor's first bucket
                self.qsgd_bucket = int(comp.bucket_size)
                self.ks, first = [], 0
                for n in layout.numels:
                    self.ks.append(first)
                    first += -(-n // self.qsgd_bucket)
                self.qsgd_nbuckets = first
            slot_bytes = Cn.quant_slot_bytes(self.codec, layout.total, nseg, owner.world_size if self.alltoall else 0,
                                             self.qsgd_nbuckets)
            self.recv = None
            if (owner.nvls and not self.alltoall and owner._virtual is None and self.codec != X.CODEC["qsgdx"]
                    and owner.world_size >= max(2, owner.nvls_min_world)):
                from ..parallel.nvls import NvlsBuffer

                stride = (slot_bytes + 255) // 256 * 256
                buf = NvlsBuffer.create(2 * owner.world_size * stride // 4, owner.group, device)   # collective
                if buf is not None:
                    self.recv = (buf, stride)
        self.clip = kind == "sparse" and bool(getattr(owner.memory, "gradient_clipping", False))
        # pipelined all-gather mode (encode of chunk c + 1 next to the pull of chunk c): same decision on every rank
        self.pipeline = None
        if (kind == "quant" and owner.pipeline and not self.alltoall and self.recv is None and owner._virtual is None):
            self.pipeline = X.pipeline_plan(layout.total, owner.world_size, self.codec, force=owner.pipeline == "force")
        heap_bytes = 2 * ((slot_bytes + 255) // 256 * 256) + 8192 + (16 * nseg + 1024 if self.clip else 0)
        self.heap = owner._make_heap(layout.key(), heap_bytes)
        self.channel = X.ExchangeChannel(self.heap, slot_bytes, nseg, owner.timeout_ms, owner.comm_sms, clip=self.clip)
        self.segs = X.segments_to_device(layout, self.ks, device)
        # the sparse kernel zeroes the output while it reads the gradient: when both alias (in-place
        # exchange) the accumulator is where later passes re-read the values, so it always exists there
        need_acc = owner._needs_acc or kind == "sparse"
        self.acc = torch.zeros(layout.total, dtype=torch.float32, device=device) if need_acc else None
        self.u = torch.zeros(layout.total, dtype=torch.float32, device=device) if owner._needs_u else None
        self.mom = torch.zeros(layout.total, dtype=torch.float32, device=device) if owner._needs_mom else None
        self.seed = _name_seed(owner.seed, "|".join(layout.names[:4]) + str(layout.total))


class FusedExchange(Communicator):
    def __init__(self, compressor, memory, world_size, mode="allgather", seed=0, timeout_ms=10000.0, comm_sms=None,
                 group=None, inplace=True, max_ratio=0.25, exact=True, rank=None, monitor=None, nvls=False,
                 nvls_min_world=4, overlap_sms=32, arena_mb=64, store=None, split_overlap=False, pipeline=True):
        """``comm_sms``: SMs an exchange may use when nothing else runs (None: all of them).  ``overlap_sms``: SMs
        of an exchange that runs next to the backward pass (launched from a gradient hook: ``send_step``, the
        bucketed ``DistributedOptimizer``, the DDP hook); the rest stays with backward.  With ``split_overlap`` such an
        exchange is two launches: compress + publish at full width (short, HBM bound), then pull + decode on
        ``overlap_sms`` SMs; measured on BERT-large it loses to the single capped launch (a full-width cooperative
        launch has to wait until backward's kernels have drained), so it is off by default.  ``arena_mb``: size of
        the symmetric heaps the plans are carved from.  ``store``: a ``torch.distributed`` store through which the
        ranks tell each other about a failed exchange (``agree`` / ``recover``)."""
        super().__init__(compressor, memory, world_size)
        self.mode = mode
        self.overlap_sms = overlap_sms
        self.split_overlap = bool(split_overlap)
        # quantised all-gather exchanges of 32 Mi elements and more: encode chunk c + 1 while chunk c is pulled
        # (False: phase by phase; "force": also for small buffers and a single rank, for tests)
        self.pipeline = pipeline
        self.arena_bytes = int(arena_mb * (1 << 20))
        self._arena = None
        self._side_stream = None
        self.store = store
        self._epoch = 0
        # push transport for the quantised codecs in all-gather mode: encoded slots are replicated into every
        # GPU's receive area with multimem.st and decoded from local memory (opt-in; needs NVSwitch multicast)
        self.nvls = bool(nvls)
        self.nvls_min_world = int(nvls_min_world)
        self.seed = int(seed)
        self.timeout_ms = float(timeout_ms)
        self.comm_sms = comm_sms
        self.group = group
        self.inplace = inplace
        self.max_ratio = max_ratio
        self.exact = exact
        self.monitor = monitor   # optional utils.faults.HeartbeatMonitor: checked before every launch
        self.nvtx = os.environ.get("GRACE_NVTX", "0") not in ("", "0")   # NVTX range around every exchange
        self.device = None
        self._rank = rank
        self._plans: Dict[tuple, _Plan] = {}
        self._single_layouts = {}
        self._virtual = None
        self._fallback = Allgather(compressor, memory, world_size)
        # what CPU tensors (and pairs without a kernel) go through: the library communicator, or - attach_host() -
        # the host engine of the same protocol, which itself falls back to the library path
        from ..utils.faults import FaultPlan

        self._faults = FaultPlan.from_env()
        self._resolve()

    # ------------------------------------------------------------------
    def _resolve(self):
        comp, mem = self.compressor, self.memory
        self._kind = None
        self._codec = None
        self._needs_acc = isinstance(mem, (M_.ResidualMemory, M_.EFSignSGDMemory, M_.DgcMemory))
        self._needs_u = isinstance(mem, M_.DgcMemory)
        self._needs_mom = isinstance(comp, C_.SignumCompressor)
        from ..ops.exchange import CODEC

        if isinstance(mem, M_.PowerSGDMemory) or isinstance(comp, C_.PowerSGDCompressor):
            self._kind = "powersgd"
        elif isinstance(comp, (C_.TopKCompressor, C_.DgcCompressor, C_.ThresholdCompressor, C_.RandomKCompressor)):
            if isinstance(mem, M_.DgcMemory) and isinstance(comp, (C_.ThresholdCompressor, C_.RandomKCompressor)):
                self._kind = None
            elif isinstance(mem, (M_.NoneMemory, M_.ResidualMemory, M_.DgcMemory)):
                self._kind = "sparse"
        elif isinstance(mem, (M_.NoneMemory, M_.ResidualMemory, M_.EFSignSGDMemory)):
            table = [
                (C_.QSGDCompressor, "qsgd"), (C_.TernGradCompressor, "terngrad"), (C_.NaturalCompressor, "natural"),
                (C_.U8bitCompressor, "u8bit"), (C_.SignSGDCompressor, "sign"), (C_.SignumCompressor, "sign"),
                (C_.EFSignSGDCompressor, "efsign"), (C_.OneBitCompressor, "onebit"), (C_.FP16Compressor, "fp16"),
                (C_.NoneCompressor, "fp32"),
            ]
            for cls, key in table:
                if isinstance(comp, cls):
                    self._codec = CODEC[key]
                    self._kind = "quant"
                    break
            if isinstance(comp, C_.QSGDCompressor) and (comp.bucket_size != 128 or comp.quantum_num >= 128):
                # the general form: int16 codes, one norm per bucket of each tensor (all-gather mode, pull transport)
                if comp.bucket_size >= 4 and comp.bucket_size % 4 == 0 and comp.quantum_num < 32768:
                    self._codec = CODEC["qsgdx"]
                else:
                    self._kind = None

    def attach_host(self, host) -> "FusedExchange":
        """Route what the kernels do not take (CPU tensors above all) through ``host`` (a ``HostExchange`` built
        for the same compressor and memory objects) instead of the library communicator."""
        self._fallback = host
        return self

    def supported(self, tensor: torch.Tensor) -> bool:
        if self._kind == "powersgd":
            return tensor.is_cuda and int(getattr(self.compressor, "rank", 1)) <= 16
        return self._kind in ("sparse", "quant") and tensor.is_cuda

    # ------------------------------------------------------------------
    def _make_heap(self, key, nbytes):
        """A range of the communicator's arena (created, collectively, on first use)."""
        from ..parallel.symm import SymmetricHeap

        if self._virtual is not None:
            return self._virtual.heap_for(key, nbytes, self._rank)
        if self._arena is None:
            self._arena = _Arena(lambda n: SymmetricHeap.create(n, group=self.group, device=self.device),
                                 self.arena_bytes)
        return self._arena.carve(nbytes)

    def prepare(self, named_tensors):
        """Create the plans of single tensors now, in name order, so that no allocation and no host collective
        is left for the first backward pass (where gradient hooks may fire in any order).  ``named_tensors``:
        iterable of ``(name, tensor)``; tensors the fused path does not cover are skipped."""
        from ..ops.exchange import FlatLayout

        for name, t in sorted(((n, t) for n, t in named_tensors), key=lambda kv: kv[0]):
            if not self.supported(t):
                continue
            if self.device is None:
                self.device = t.device
            lkey = (name, t.numel(), tuple(t.shape))
            layout = self._single_layouts.get(lkey)
            if layout is None:
                layout = self._single_layouts[lkey] = FlatLayout.single(name, t.numel(), t.shape)
            self._plan(layout)

    def prepare_layouts(self, layouts, device):
        """Same for whole buckets (``FlatParams.buckets``), in the order given."""
        if self.device is None:
            self.device = torch.device(device)
        for layout in layouts:
            self._plan(layout)

    def _comm_stream(self):
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device, priority=-1)
        return self._side_stream

    def close(self):
        """Tear down: wait for this rank's launches, meet the other ranks, unmap and free the arena.
        Error-feedback state goes with the plans; take ``state_dict()`` first to keep it."""
        if self.device is not None and torch.device(self.device).type == "cuda":
            torch.cuda.synchronize(self.device)
        if (self._virtual is None and self._arena is not None and dist.is_available() and dist.is_initialized()
                and self.world_size > 1):
            dist.barrier(group=self.group)
        self._plans.clear()
        self._single_layouts.clear()
        if self._arena is not None:
            self._arena.close()
            self._arena = None
        if hasattr(self._fallback, "close"):   # an attached host engine
            self._fallback.close()

    def _plan(self, layout) -> _Plan:
        key = getattr(layout, "_key", None)
        if key is None:
            key = layout._key = layout.key()
        plan = self._plans.get(key)
        if plan is None:
            if self._kind == "powersgd":
                from ..ops.lowrank import LowRankPlan

                plan = LowRankPlan(self._make_heap, layout, layout.shape_list(), int(self.compressor.rank),
                                   self.world_size, isinstance(self.memory, M_.PowerSGDMemory), self.device,
                                   seed=self.seed, timeout_ms=self.timeout_ms, sm_limit=self.comm_sms)
                plan.kind = "powersgd"
            else:
                plan = _Plan(self, layout, self._kind)
            pending = getattr(self, "_pending_state", None)
            if pending:  # a checkpoint was loaded before this layout was first used
                self._restore_plan(plan, pending)
            self._plans[key] = plan
        return plan

    def _memory_coeffs(self, plan: _Plan):
        mem = self.memory
        first = plan.steps == 0
        if isinstance(mem, M_.ResidualMemory):
            return (0.0, 1.0) if first else (float(mem.beta), float(mem.gamma))
        if isinstance(mem, M_.EFSignSGDMemory):
            return (0.0, 1.0) if first else (1.0, float(mem.learning_rate))
        return 0.0, 1.0

    def _launch(self, plan: _Plan, g: torch.Tensor, out: torch.Tensor, phases: int, seq: Optional[int] = None,
                sm_limit: Optional[int] = None) -> int:
        from ..ops import exchange as X

        grid = None if sm_limit is None else plan.channel.max_grid(plan.kind, sm_limit)

        comp = self.compressor
        scale = (1.0 / self.world_size) if comp.average else 1.0
        beta, gamma = self._memory_coeffs(plan)
        plan.channel.poll()
        if plan.kind == "sparse" and plan.clip and phases == X.PHASE_ALL:
            phases |= X.PHASE_CLIP   # one launch: sums of squares, their exchange, clamp, compress, exchange
        if self._faults.action and (phases & X.PHASE_PUBLISH) and self._faults.hits(
                "skip_publish", plan.heap.rank, plan.steps):
            phases &= ~X.PHASE_PUBLISH  # host-side fault injection: this rank "forgets" to publish
        if plan.kind == "sparse":
            seq = X.run_sparse(
                plan.channel, plan.layout, plan.segs, g, plan.acc, plan.u, out, mode=plan.mode, cap=plan.cap,
                beta=beta, gamma=gamma, momentum=float(getattr(self.memory, "momentum", 0.0)),
                threshold=float(getattr(comp, "threshold", 0.0)), scale=scale, levels=3 if self.exact else 2,
                phases=phases, seq=seq, kprefix=plan.kprefix, seg_seed=plan.seg_seed, rk_step=plan.steps,
                clip=plan.clip, strict=bool(getattr(comp, "strict", False)), tile_decode=plan.tile, grid=grid)
        else:
            seq = X.run_quant(
                plan.channel, plan.layout, plan.segs, g, plan.acc, plan.mom, out, codec=plan.codec,
                quantum=int(getattr(comp, "quantum_num", 0)), deterministic=bool(getattr(comp, "deterministic", False)),
                first_step=plan.steps == 0, beta=beta, gamma=gamma, mom_beta=float(getattr(comp, "momentum", 0.0)),
                lr=float(getattr(comp, "learning_rate", 1.0)), scale=scale, seed=plan.seed, step=plan.steps,
                phases=phases | (X.PHASE_REDUCE if (plan.alltoall and phases == X.PHASE_ALL) else 0), seq=seq,
                recv=plan.recv, alltoall=plan.alltoall, grid=grid, qsgd_bucket=plan.qsgd_bucket,
                qsgd_nbuckets=plan.qsgd_nbuckets,
                pipeline=plan.pipeline if (phases == X.PHASE_ALL and plan.channel.chunk_ready_off) else None)
        return seq

    # ------------------------------------------------------------------
    def step_flat(self, flat: torch.Tensor, layout, out: Optional[torch.Tensor] = None,
                  sm_limit: Optional[int] = None) -> torch.Tensor:
        """Exchange a whole flat buffer of named gradients in one launch (on the current stream).
        ``sm_limit`` caps the grid of this launch (an exchange that runs next to backward)."""
        from ..ops.exchange import PHASE_ALL

        if self.device is None:
            self.device = flat.device
        if self.monitor is not None:
            self.monitor.beat(force=False)
            dead = self.monitor.dead_ranks()
            if dead:
                raise RuntimeError("grace: ranks %s stopped sending heartbeats; not launching an exchange "
                                   "that could only time out" % dead)
        plan = self._plan(layout)
        out = flat if out is None else out
        from ..utils import timeline

        tl = timeline.active()
        tok = None
        if tl is not None:
            tok = tl.begin(layout.names[0] if len(layout.names) == 1 else "%d tensors" % len(layout.names),
                           "fused." + plan.kind, device=flat.is_cuda, numel=sum(layout.numels),
                           compressor=type(self.compressor).__name__, payload_bytes=self._payload_bytes(plan))
        nvtx = self.nvtx and flat.is_cuda
        if nvtx:
            torch.cuda.nvtx.range_push("grace.exchange.%s" % plan.kind)
        self._stats["dense_bytes"] += 4 * sum(layout.numels)
        self._stats["payload_bytes"] += self._payload_bytes(plan)
        if plan.kind == "powersgd":
            if plan.matrices:
                plan.channel.poll()
                plan.launch(flat, out, sm_limit=sm_limit)
            plan.launch_dense(flat, out, sm_limit=sm_limit)
        elif sm_limit is not None and self.split_overlap:
            # next to backward: the compress half is HBM bound and short, so it runs at full width; the exchange half
            # mostly waits for NVLink, so it keeps to a few SMs and leaves the rest to the backward kernels
            from ..ops.exchange import PHASE_CLIP, PHASE_COMPRESS, PHASE_EXCHANGE, PHASE_PUBLISH, PHASE_REDUCE

            first = PHASE_COMPRESS | PHASE_PUBLISH | (PHASE_CLIP if getattr(plan, "clip", False) else 0)
            second = PHASE_EXCHANGE | (PHASE_REDUCE if getattr(plan, "alltoall", False) else 0)
            seq = self._launch(plan, flat, out, first)
            self._launch(plan, flat, out, second, seq=seq, sm_limit=sm_limit)
        else:
            self._launch(plan, flat, out, PHASE_ALL, sm_limit=sm_limit)
        plan.steps += 1
        self._stats["steps"] += 1
        if nvtx:
            torch.cuda.nvtx.range_pop()
        if tok is not None:
            tl.end(tok)
        return out

    def _payload_bytes(self, plan) -> int:
        """Bytes this rank publishes per exchange of ``plan`` (what a peer pulls)."""
        if plan.kind == "sparse":
            return 8 * (sum(plan.ks) if plan.ks else plan.cap)
        if plan.kind == "quant":
            return int(plan.channel.slot_bytes)
        dense = 4 * plan.dense_layout.total if plan.dense else 0
        return 4 * (plan.p_floats + plan.q_floats) * self.compressor.rank // 16 + dense

    def _prepare(self, tensor: torch.Tensor):
        """The gradient as a flat, aligned buffer the kernels can read: fp32, bf16 and fp16 tensors are taken as
        they are (the kernels convert on load); anything else is cast to fp32 first.  The low-rank kernel reads
        fp32 only (its TMA tensor maps are typed)."""
        flat = tensor.detach().reshape(-1)
        keep = (torch.float32,) if self._kind == "powersgd" else (torch.float32, torch.bfloat16, torch.float16)
        if flat.dtype not in keep:
            flat = flat.float()
        if not flat.is_contiguous() or flat.data_ptr() % 16 != 0:
            flat = flat.contiguous().clone()
        return flat

    def step(self, tensor: torch.Tensor, name: str, sm_limit: Optional[int] = None) -> torch.Tensor:
        if not self.supported(tensor):
            return self._fallback.step(tensor, name)
        from ..ops.exchange import FlatLayout

        flat = self._prepare(tensor)
        same = flat.data_ptr() == tensor.data_ptr()
        if self._kind == "sparse" and flat.dtype != torch.float32:
            out = torch.empty(flat.shape, dtype=torch.float32, device=flat.device)   # the scatter-add needs fp32 words
        else:
            out = flat if (self.inplace and same) else torch.empty_like(flat)
        lkey = (name, flat.numel(), tuple(tensor.shape))
        layout = self._single_layouts.get(lkey)
        if layout is None:
            layout = self._single_layouts[lkey] = FlatLayout.single(name, flat.numel(), tensor.shape)
        self.step_flat(flat, layout, out, sm_limit=sm_limit)
        return out.view(tensor.shape).to(tensor.dtype)

    # split-phase (the reference's Horovod flavour, grace_dl/torch/__init__.py:50-58): the exchange is launched
    # from the gradient hook on a high-priority side stream with a capped grid, so it runs next to the rest of
    # backward; receive_step makes the caller's stream wait for it
    def send_step(self, tensor: torch.Tensor, name: str):
        if not self.supported(tensor):
            return self._fallback.send_step(tensor, name)
        if self.device is None:
            self.device = tensor.device
        side = self._comm_stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            out = self.step(tensor, name, sm_limit=self.overlap_sms)
            ev = torch.cuda.Event()
            ev.record(side)
        return ("fused", out, ev), None

    def receive_step(self, handles, ctx) -> torch.Tensor:
        if isinstance(handles, tuple) and len(handles) == 3 and handles[0] == "fused":
            _, out, ev = handles
            cur = torch.cuda.current_stream()
            cur.wait_event(ev)
            out.record_stream(cur)
            return out
        return self._fallback.receive_step(handles, ctx)

    def send_receive(self, tensors, name, ctx):
        return self._fallback.send_receive(tensors, name, ctx)

    def reset(self):
        """After a ``GraceCommError``: clear flags, sequence numbers and scratch of every plan.
        Call it on every rank, then synchronise the ranks on the host (``dist.barrier()``) before
        the next exchange.  Error-feedback state is kept."""
        for plan in self._plans.values():
            if plan.kind == "powersgd":
                if plan.matrices:
                    plan.channel.reset()
                if plan.dense:
                    plan.dense_channel.reset()
            else:
                plan.channel.reset()

    def agree(self, local_error: Optional[BaseException] = None, timeout_s: float = 30.0):
        """Step-boundary vote through the store: every rank posts whether its exchanges failed and reads the
        others' votes.  Returns the sorted list of ranks that reported a failure (empty: all healthy), the same
        list on every rank, so that either all of them call ``recover()`` or none does.  Needs ``store``."""
        if self.store is None:
            raise RuntimeError("agree() needs a store (FusedExchange(..., store=...))")
        board = self._error_board()
        failed = local_error is not None
        if not failed:
            try:
                self.check()
            except RuntimeError as e:   # GraceCommError included
                local_error, failed = e, True
        return board.vote(self._epoch, failed, timeout_s=timeout_s,
                          info=str(local_error)[:200] if failed else "")

    def recover(self, timeout_s: float = 30.0):
        """After a failed exchange, on every rank: (1) wait for this rank's kernels (their waits are bounded, so
        this returns) - from then on this rank writes no flag of a peer any more; (2) meet the other ranks;
        (3) clear flags, sequence numbers and scratch of every plan; (4) meet again, so that nobody launches
        before every pad is clean.  The meetings go through the store when one is attached, else through
        process-group barriers.  Error-feedback state, warm starts and step counters are kept; the next exchange
        starts from sequence 1 on every rank."""
        if self.device is not None and torch.device(self.device).type == "cuda":
            torch.cuda.synchronize(self.device)
        real = self._virtual is None and self.world_size > 1

        def meet(tag):
            if not real:
                return
            if self.store is not None:
                self._error_board().barrier(self._epoch, timeout_s=timeout_s, tag=tag)
            elif dist.is_available() and dist.is_initialized():
                dist.barrier(group=self.group)

        meet("quiet")
        self.reset()
        meet("clean")
        self._epoch += 1

    def _error_board(self):
        from ..utils.faults import ErrorBoard

        if getattr(self, "_board", None) is None:
            self._board = ErrorBoard(self.store, self._host_rank(), self.world_size)
        return self._board

    def _host_rank(self) -> int:
        if self._rank is not None:
            return int(self._rank)
        return dist.get_rank(self.group) if dist.is_available() and dist.is_initialized() else 0

    def check(self):
        """Block until every launched exchange finished; raise on failure."""
        for plan in self._plans.values():
            if plan.kind == "powersgd":
                plan.check()
            else:
                plan.channel.check()
        if hasattr(self._fallback, "check"):   # an attached host engine
            self._fallback.check()

    # ------------------------------------------------------------------
    def state_dict(self):
        if not self._plans:
            return self._fallback.state_dict()
        residuals, gradients, momentums = {}, {}, {}
        q_memory = {}
        for plan in self._plans.values():
            lay = plan.layout
            if plan.kind == "powersgd":
                if plan.acc is not None:
                    for n, t in lay.slices(plan.acc).items():
                        residuals[n] = t.clone()
                if plan.matrices:
                    q_memory.update(plan.q_memory())
                continue
            if plan.acc is not None:
                target = gradients if plan.u is not None else residuals
                for n, t in lay.slices(plan.acc).items():
                    target[n] = t.clone()
            if plan.u is not None:
                for n, t in lay.slices(plan.u).items():
                    residuals[n] = t.clone()
            if plan.mom is not None:
                for n, t in lay.slices(plan.mom).items():
                    momentums[n] = t.clone()
        mem = {"residuals": residuals}
        if gradients:
            mem["gradients"] = gradients
        comp = self.compressor.state_dict()
        if momentums:
            comp["momentums"] = momentums
        if q_memory:
            comp["q_memory"] = q_memory
        steps = {"|".join(map(str, k[1])) + ":" + "|".join(k[0][:2]): p.steps for k, p in self._plans.items()}
        return {"compressor": comp, "memory": mem, "world_size": self.world_size, "fused_steps": steps}

    def load_state_dict(self, state):
        self._pending_state = state
        self._fallback.load_state_dict(state)
        for plan in self._plans.values():
            self._restore_plan(plan, state)

    def _restore_plan(self, plan: _Plan, state):
        mem = state.get("memory", {})
        lay = plan.layout
        if plan.kind == "powersgd":
            if plan.acc is not None:
                for n, t in lay.slices(plan.acc).items():
                    if n in mem.get("residuals", {}):
                        t.copy_(mem["residuals"][n].reshape(-1))
            if plan.matrices:
                plan.load_q_memory(state.get("compressor", {}).get("q_memory", {}))
            return
        src_acc = mem.get("gradients" if plan.u is not None else "residuals", {})
        if plan.acc is not None:
            for n, t in lay.slices(plan.acc).items():
                if n in src_acc:
                    t.copy_(src_acc[n].reshape(-1))
                    plan.steps = max(plan.steps, 1)
        if plan.u is not None:
            for n, t in lay.slices(plan.u).items():
                if n in mem.get("residuals", {}):
                    t.copy_(mem["residuals"][n].reshape(-1))
        if plan.mom is not None:
            for n, t in lay.slices(plan.mom).items():
                if n in state.get("compressor", {}).get("momentums", {}):
                    t.copy_(state["compressor"]["momentums"][n].reshape(-1))
                    plan.steps = max(plan.steps, 1)
        key = "|".join(map(str, lay.key()[1])) + ":" + "|".join(lay.key()[0][:2])
        if key in state.get("fused_steps", {}):
            plan.steps = int(state["fused_steps"][key])


class VirtualWorld:
    """W ``FusedExchange`` objects on ONE GPU, stepped phase by phase.

    Ranks never wait on each other inside a kernel: all ranks run
    compress+publish first, then all ranks run exchange, each as its own
    launch on the same stream.  The protocol (flags, slots, acknowledgements,
    sequence numbers) and the kernels are the ones a real multi-GPU run uses.
    """

    def __init__(self, world: int, make_comm, device=None):
        self.world = world
        self.device = torch.device(device if device is not None else "cuda")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self._heaps = {}
        self._arena = None
        self.arena_bytes = 64 << 20
        self.comms: List[FusedExchange] = []
        for r in range(world):
            c = make_comm(r)
            c._virtual = self
            c._rank = r
            c.device = self.device
            self.comms.append(c)

    def heap_for(self, key, nbytes, rank):
        """Range ``key`` of the world's arena, as seen by virtual rank ``rank`` (carved once for all W ranks)."""
        from ..parallel.symm import SymmetricHeap

        if key not in self._heaps:
            if self._arena is None:
                self._arena = _Arena(lambda n: _VirtualSegment(SymmetricHeap.virtual(n, self.world, self.device)),
                                     self.arena_bytes)
            self._heaps[key] = self._arena.carve(nbytes)
        return self._heaps[key][rank]

    def step_flat(self, flats: Sequence[torch.Tensor], layout, outs: Optional[Sequence[torch.Tensor]] = None):
        from ..ops.exchange import PHASE_COMPRESS, PHASE_EXCHANGE, PHASE_PUBLISH

        outs = list(outs) if outs is not None else list(flats)
        plans = [c._plan(layout) for c in self.comms]
        if plans[0].kind == "powersgd":
            if plans[0].matrices:
                seqs = [p.launch(g, o, part=1) for p, g, o in zip(plans, flats, outs)]
                for part in (2, 3):
                    for p, g, o, s in zip(plans, flats, outs, seqs):
                        p.launch(g, o, part=part, seq=s)
            if plans[0].dense:
                seqs = [p.launch_dense(g, o, PHASE_COMPRESS | PHASE_PUBLISH) for p, g, o in zip(plans, flats, outs)]
                for p, g, o, s in zip(plans, flats, outs, seqs):
                    p.launch_dense(g, o, PHASE_EXCHANGE, seq=s)
            for p in plans:
                p.steps += 1
            return outs
        seqs = [None] * len(plans)
        if getattr(plans[0], "clip", False):   # every rank's sums of squares first: compress reads all of them
            from ..ops.exchange import PHASE_CLIP

            seqs = [c._launch(p, g, o, PHASE_CLIP) for c, p, g, o in zip(self.comms, plans, flats, outs)]
        seqs = [c._launch(p, g, o, PHASE_COMPRESS | PHASE_PUBLISH, seq=s)
                for c, p, g, o, s in zip(self.comms, plans, flats, outs, seqs)]
        if getattr(plans[0], "alltoall", False):
            from ..ops.exchange import PHASE_REDUCE

            for c, p, g, o, s in zip(self.comms, plans, flats, outs, seqs):
                c._launch(p, g, o, PHASE_REDUCE, seq=s)
        for c, p, g, o, s in zip(self.comms, plans, flats, outs, seqs):
            c._launch(p, g, o, PHASE_EXCHANGE, seq=s)
            p.steps += 1
        return outs

    def step(self, tensors: Sequence[torch.Tensor], name: str):
        from ..ops.exchange import FlatLayout

        flats = [c._prepare(t) for c, t in zip(self.comms, tensors)]
        outs = [torch.empty_like(f) for f in flats]
        self.step_flat(flats, FlatLayout.single(name, flats[0].numel(), tensors[0].shape), outs)
        return [o.view(t.shape) for o, t in zip(outs, tensors)]

    def check(self):
        for c in self.comms:
            c.check()
