"""Launch plans for the fused exchange kernels.

A ``FlatLayout`` describes how named gradients sit in one flat fp32 buffer
(every tensor starts on a 128-element boundary).  An ``ExchangeChannel`` owns
what one stream of exchanges needs on the symmetric heap: the ready/ack flag
pads and two send slots (double buffered by sequence parity), plus the local
scratch (histograms, per-segment state, barrier word, status block) and the
error-feedback arenas.  ``run_sparse`` / ``run_quant`` fill the argument block
and launch the cooperative kernel on the current stream.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import native
from ..parallel.symm import SymmetricHeap

PHASE_COMPRESS, PHASE_PUBLISH, PHASE_EXCHANGE, PHASE_ALL = 1, 2, 4, 7
PHASE_REDUCE = 8  # two-phase (alltoall) mode: reduce my chunk, re-encode, publish again
PHASE_CLIP = 16   # sparse exchange with DGC gradient clipping: per-tensor sums of squares, published before compress
GRAD_DTYPE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
SPARSE_TOPK, SPARSE_THRESHOLD, SPARSE_RANDOMK = 0, 1, 2
CODEC = {"qsgd": 0, "terngrad": 1, "natural": 2, "u8bit": 3, "sign": 4, "efsign": 5, "onebit": 6, "fp16": 7, "fp32": 8,
         "qsgdx": 9}   # QSGD with any bucket size (multiple of 4) and up to 32767 levels: int16 codes

STATUS_TEXT = {
    0: "ok", 1: "timeout at a grid barrier", 2: "timeout waiting for a peer's data",
    3: "timeout waiting for a peer's acknowledgement", 4: "send slot overflow", 5: "bad argument / corrupt index",
    6: "timeout on an mbarrier",
    7: "a bounds check of the checked build failed (detail = source line; the access was skipped)",
}
ALIGN_ELEMS = 128
GUARD_BYTES = 256
GUARD_PATTERN = 0xA5


class GraceCommError(RuntimeError):
    """A fused exchange reported a failure (bounded wait expired, bad data)."""

    def __init__(self, code: int, detail: int, seq: int, rank: int):
        self.code, self.detail, self.seq, self.rank = code, detail, seq, rank
        super().__init__(
            "fused exchange failed on rank %d at sequence %d: %s (detail=%d)"
            % (rank, seq, STATUS_TEXT.get(code, "code %d" % code), detail)
        )


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class FlatLayout:
    """Placement of named tensors in a flat buffer."""

    names: List[str]
    numels: List[int]
    offsets: List[int] = field(default_factory=list)
    total: int = 0
    shapes: Optional[List[Tuple[int, ...]]] = None   # original tensor shapes (PowerSGD needs rows x cols)

    def __post_init__(self):
        if not self.offsets:
            off = 0
            for n in self.numels:
                self.offsets.append(off)
                off += _round_up(n, ALIGN_ELEMS)
            self.total = off
        if self.total == 0 and self.numels:
            self.total = _round_up(self.offsets[-1] + self.numels[-1], ALIGN_ELEMS)
        if self.total >= 2 ** 31:
            raise ValueError("flat buffers are indexed with 31 bits; split the bucket (%d elements)" % self.total)

    @classmethod
    def single(cls, name: str, numel: int, shape=None) -> "FlatLayout":
        lay = cls([name], [numel])
        lay.shapes = [tuple(shape)] if shape is not None else None
        return lay

    @classmethod
    def from_named(cls, named: Sequence[Tuple[str, int]]) -> "FlatLayout":
        return cls([n for n, _ in named], [int(c) for _, c in named])

    def key(self) -> Tuple:
        return (tuple(self.names), tuple(self.numels))

    def shape_list(self):
        return self.shapes if self.shapes is not None else [(n,) for n in self.numels]

    def segment_bytes(self, ks: Optional[Sequence[int]] = None) -> bytes:
        ks = ks if ks is not None else [0] * len(self.names)
        return b"".join(struct.pack("<qii", off, n, k) for off, n, k in zip(self.offsets, self.numels, ks))

    def slices(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {n: flat[o : o + c] for n, o, c in zip(self.names, self.offsets, self.numels)}


class ExchangeChannel:
    """Flags + two send slots on the symmetric heap, and local scratch."""

    def __init__(self, heap: SymmetricHeap, slot_bytes: int, nseg: int, timeout_ms: float = 10000.0,
                 sm_limit: Optional[int] = None, clip: bool = False):
        C = native()
        self.heap = heap
        self.device = heap.device
        self.slot_bytes = _round_up(slot_bytes, 256)
        self.flags_off = heap.alloc(2 * C.MAX_WORLD * 8)
        self.ready_off = self.flags_off
        self.ack_off = self.flags_off + C.MAX_WORLD * 8
        # GRACE_GUARD=1: poison-filled guard bands around both send slots, checked by check()
        # (stands in for a memory checker: a kernel writing outside its slot is caught on the host)
        self.guard = bool(os.environ.get("GRACE_GUARD")) and heap.free_bytes >= 2 * self.slot_bytes + 4 * GUARD_BYTES
        self.guard_off = []
        if self.guard:
            self.guard_off.append(heap.alloc(GUARD_BYTES))
        self.slot_off = [heap.alloc(self.slot_bytes)]
        if self.guard:
            self.guard_off.append(heap.alloc(GUARD_BYTES))
        self.slot_off.append(heap.alloc(self.slot_bytes))
        if self.guard:
            self.guard_off.append(heap.alloc(GUARD_BYTES))
            for off in self.guard_off:
                heap.view(off, GUARD_BYTES, torch.uint8).fill_(GUARD_PATTERN)
        self.ready2_off = heap.alloc(C.MAX_WORLD * 8) if heap.free_bytes >= C.MAX_WORLD * 8 + 256 else 0
        # pipelined quantised exchange: one "published" flag per rank and chunk, and the queue / chunk counters
        chunk_flags = C.MAX_WORLD * C.PIPE_MAX_CHUNKS * 8
        self.chunk_ready_off = heap.alloc(chunk_flags) if heap.free_bytes >= chunk_flags + 256 else 0
        self.pipe = torch.zeros(1 + C.PIPE_MAX_CHUNKS, dtype=torch.int32, device=heap.device)
        # DGC gradient clipping: every rank publishes its per-tensor sums of squares (two parities) + a flag pad
        self.clip_off = self.clip_ready_off = 0
        self.clip_sq = None
        if clip:
            self.clip_ready_off = heap.alloc(C.MAX_WORLD * 8)
            self.clip_off = heap.alloc(2 * max(1, nseg) * 8)
            self.clip_sq = torch.zeros(max(1, nseg), dtype=torch.float64, device=heap.device)
        self.seq = 0
        self._grids = {}
        self.timeout_ns = int(timeout_ms * 1e6)
        self.sm_limit = sm_limit or 0
        dev = self.device
        self.barrier = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(32, dtype=torch.int32, device=dev)   # [0..3] error block, [8..] optional phase counters
        self.status_host = torch.zeros(32, dtype=torch.int32).pin_memory() if torch.cuda.is_available() else None
        self.status_event: Optional[int] = None    # event of the last launch (None: nothing launched since a reset)
        self.status_every = max(1, int(os.environ.get("GRACE_STATUS_EVERY", "8")))   # launches per status copy for poll()
        self._since_copy = 0
        self._copy_event: Optional[int] = None     # plain CUDA events (handles), created on first use
        self._last_event: Optional[int] = None
        self._copy_pending = False
        # radix-select histograms: first level, hinted second level (zero between launches), then one hint word per
        # segment (the first-level pivot bin of the previous launch, -1 = none; a speed hint only)
        self._hist_segs = max(1, nseg)
        self.hist = torch.zeros(self._hist_segs * (2 * 4096 + 1), dtype=torch.int32, device=dev)
        self.hist[2 * 4096 * self._hist_segs:] = -1
        self.sparse_state = torch.zeros((max(1, nseg) + 1) * (C.SPARSE_STATE_BYTES // 4), dtype=torch.int32, device=dev)
        self.cand = None  # candidate list of the fast top-k path, allocated by run_sparse on first use
        self._tile = None  # scratch of the tile-bucketed decode: (key, buffers) or (key, None) when not worthwhile
        self.quant_stats = torch.zeros(max(1, nseg) * C.QUANT_STATS_BYTES, dtype=torch.uint8, device=dev)

    def next_seq(self) -> int:
        self.seq += 1
        return self.seq

    def max_grid(self, kind: str, sm_limit: Optional[int] = None) -> int:
        """Largest co-resident grid of a kernel family on this device (cached).  ``sm_limit`` overrides the
        channel's own limit for one launch (a capped grid leaves SMs to the backward pass it overlaps with)."""
        limit = self.sm_limit if sm_limit is None else int(sm_limit)
        g = self._grids.get((kind, limit))
        if g is None:
            C = native()
            fn = C.sparse_max_grid if kind == "sparse" else C.quant_max_grid
            g = fn(self.heap.device.index, limit)
            self._grids[(kind, limit)] = g
        return g

    def tile_scratch(self, total: int):
        """Local scratch of the tile-ordering step of the sparse exchange (counters, cursors, scan words)."""
        if self._tile is None or self._tile[0] != total:
            tiles = -(-total // TILE_ELEMS)
            dev = self.device
            self._tile = (total, (torch.zeros(tiles + 1, dtype=torch.int32, device=dev),
                                  torch.empty(tiles, dtype=torch.int32, device=dev),
                                  torch.empty(self.max_grid("sparse", 0), dtype=torch.int32, device=dev)))
        return self._tile[1]

    def slot_view(self, seq: int, numel: int, dtype, byte_offset: int = 0, rank: Optional[int] = None):
        return self.heap.view(self.slot_off[seq & 1] + byte_offset, numel, dtype, rank)

    # -- error surface ----------------------------------------------------
    def post_status(self):
        """Mark the launch just queued on the current stream (a plain CUDA event, no sync).  Every
        ``status_every``-th launch also queues a copy of the status block to pinned memory, which is what ``poll()``
        looks at; ``check()`` fetches the block itself, so it never depends on those copies.  (A copy and a
        framework event per launch cost more host time than the launch of a small exchange.)"""
        C = native()
        if self._last_event is None:
            self._last_event = C.event_create()
        C.event_record(self._last_event, _stream_ptr(self.device.index))
        self.status_event = self._last_event
        self._since_copy += 1
        if self._since_copy >= self.status_every:
            self._since_copy = 0
            self.status_host.copy_(self.status, non_blocking=True)
            if self._copy_event is None:
                self._copy_event = C.event_create()
            C.event_record(self._copy_event, _stream_ptr(self.device.index))
            self._copy_pending = True

    def poll(self):
        """Raise if a launch whose status has already reached the host reported a failure; never blocks."""
        if self._copy_pending and native().event_query(self._copy_event):
            self._copy_pending = False
            self._raise_if_failed()

    def check(self):
        """Synchronise with the last launch, fetch its status block and raise if it failed."""
        if self.status_event is not None:
            C = native()
            C.event_synchronize(self.status_event)
            if self._copy_pending:
                C.event_synchronize(self._copy_event)   # an older copy must not land after the one below
                self._copy_pending = False
            self.status_host.copy_(self.status)
            self._since_copy = 0
            self._raise_if_failed()
        if self.guard:
            self.verify_guards()

    def __del__(self):
        try:
            C = native()
            for ev in (self._last_event, self._copy_event):
                if ev is not None:
                    C.event_destroy(ev)
        except Exception:
            pass

    def verify_guards(self):
        for off in self.guard_off:
            band = self.heap.view(off, GUARD_BYTES, torch.uint8)
            if not bool((band == GUARD_PATTERN).all()):
                raise RuntimeError("grace: guard band at heap offset %d was overwritten (a kernel wrote outside "
                                   "its send slot)" % off)

    def dropped(self) -> int:
        self.check()
        return int(self.status_host[3])

    def _raise_if_failed(self):
        code = int(self.status_host[0])
        if code != 0:
            detail, seq = int(self.status_host[1]), int(self.status_host[2])
            err = GraceCommError(code, detail, seq, self.heap.rank)
            if code == 7:   # checked build: which kernel and which index
                err.kernel = int(self.status_host[4])
                err.index = int(self.status_host[5]) | (int(self.status_host[6]) << 32)
                err.args = (err.args[0] + " [kernel %d, index %d]" % (err.kernel, err.index),)
            raise err

    def reset(self):
        """Clear flags and status after an error (call on every rank, then barrier)."""
        C = native()
        torch.cuda.synchronize(self.device)
        self.heap.view(self.flags_off, 2 * C.MAX_WORLD, torch.int64).zero_()
        if self.ready2_off:
            self.heap.view(self.ready2_off, C.MAX_WORLD, torch.int64).zero_()
        if self.chunk_ready_off:
            self.heap.view(self.chunk_ready_off, C.MAX_WORLD * C.PIPE_MAX_CHUNKS, torch.int64).zero_()
        if self.clip_ready_off:
            self.heap.view(self.clip_ready_off, C.MAX_WORLD, torch.int64).zero_()
            self.clip_sq.zero_()
        self.status.zero_()
        self.hist.zero_()
        self.hist[2 * 4096 * self._hist_segs:] = -1
        self.sparse_state.zero_()
        self.quant_stats.zero_()
        self.seq = 0
        self.status_event = None
        self._since_copy = 0
        self._copy_pending = False
        if self.status_host is not None:
            self.status_host.zero_()
        torch.cuda.synchronize(self.device)


def _stream_ptr(device_index: Optional[int] = None) -> int:
    """Handle of the current stream of a device (the short way: ``torch.cuda.current_stream()`` builds a stream
    object and resolves the device on every call, ten times the cost)."""
    if device_index is None:
        device_index = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(device_index)


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


# Tile-ordered sparse exchange: the sender orders its (value, index) list by 8192-element output tile and
# publishes a directory of tile offsets; receivers build whole output tiles in shared memory (ranks in order)
# and write them once, densely, instead of scatter-adding every entry into global memory.  It pays once the
# output no longer fits the L2 cache AND the ranks together deliver a percent or two of its elements; below
# that the scattered adds are cheaper than the dense write.  Measured on one B200 with 8 lists of 256 Mi
# elements each (compress + exchange phase of one rank): 1 % per list 1.27 ms against 2.00 ms, 0.1 % per list
# 1.13 against 1.08 ms; 2 lists of 1 %: 1.15 against 1.25 ms; 8 lists of 1 % of 32 Mi: 0.29 against 0.35 ms.  GRACE_TILE_DECODE=0 turns it off, =force turns it on
# for every size.  Every rank must decide alike (the slot layout depends on it): the rule uses only the
# layout, the capacity and the world size.
_TILE_ENV = os.environ.get("GRACE_TILE_DECODE", "1")
TILE_DECODE_DEFAULT = _TILE_ENV != "0"
TILE_DECODE_MIN_ELEMS = 0 if _TILE_ENV == "force" else 1 << 24
TILE_DECODE_MIN_DENSITY = 0.0 if _TILE_ENV == "force" else 1.0 / 32     # world * capacity / elements
TILE_DECODE_MAX_DENSITY = 0.5                                            # above this the lists outweigh the tiles


def tile_decode_wanted(total: int, cap: int, world: int, mode: int) -> bool:
    if not TILE_DECODE_DEFAULT or mode == SPARSE_RANDOMK:
        return False
    if mode == SPARSE_THRESHOLD and _TILE_ENV != "force":
        # the capacity of a threshold exchange is a bound (max_ratio), not the number of entries that will travel:
        # it says nothing about the density, and the ordered copy of the list would double an already large slot
        return False
    return (total >= TILE_DECODE_MIN_ELEMS and world * cap >= TILE_DECODE_MIN_DENSITY * total
            and cap <= TILE_DECODE_MAX_DENSITY * total)


TILE_ELEMS = 8192


def sparse_capacity(layout: FlatLayout, ks: Sequence[int], mode: int, max_ratio: float = 1.0) -> int:
    if mode in (SPARSE_TOPK, SPARSE_RANDOMK):
        cap = sum(ks)
    else:
        cap = int(sum(layout.numels) * max_ratio) + 16
    return _round_up(max(cap, 16), 16)


def run_sparse(channel: ExchangeChannel, layout: FlatLayout, segs_dev: torch.Tensor, g: torch.Tensor,
               acc: Optional[torch.Tensor], u: Optional[torch.Tensor], out: Optional[torch.Tensor], *, mode: int,
               cap: int, beta: float = 1.0, gamma: float = 1.0, momentum: float = 0.0, threshold: float = 0.0,
               scale: float = 1.0, levels: int = 3, phases: int = PHASE_ALL, seq: Optional[int] = None,
               grid: Optional[int] = None, kprefix: Optional[torch.Tensor] = None,
               seg_seed: Optional[torch.Tensor] = None, rk_step: int = 0,
               clip: bool = False, strict: bool = False, tile_decode: bool = False) -> int:
    """``tile_decode``: the slot was sized with ``sparse_slot_bytes(cap, total)`` and every rank orders its list
    by output tile (see ``tile_decode_wanted``)."""
    C = native()
    heap = channel.heap
    if seq is None:
        seq = channel.next_seq()
    if grid is None:
        grid = channel.max_grid("sparse")
    td = channel.tile_scratch(layout.total) if (tile_decode and mode != SPARSE_RANDOMK) else None
    need = -(-layout.total // 2048)
    grid = max(1, min(grid, max(need, 1)))
    for t in (acc, u, out):
        if t is not None:
            assert t.dtype == torch.float32 and t.is_cuda and t.data_ptr() % 16 == 0, "fp32, cuda, 16-byte aligned"
    assert g.is_cuda and g.dtype in GRAD_DTYPE and g.data_ptr() % (16 if g.dtype == torch.float32 else 8) == 0, \
        "gradients: fp32 (16-byte aligned), bf16 or fp16 (8-byte aligned) on the GPU"
    if clip and not channel.clip_off:
        raise ValueError("this channel was built without a clipping area (ExchangeChannel(..., clip=True))")
    cand_cap = 0
    if mode == SPARSE_TOPK and levels == 3 and (phases & PHASE_COMPRESS):
        if channel.cand is None:
            channel.cand_cap = max(65536, layout.total // 8)
            channel.cand = torch.empty(2 * channel.cand_cap, dtype=torch.int32, device=channel.device)
        cand_cap = channel.cand_cap
    C.sparse_exchange(
        _ptr(g), _ptr(acc), _ptr(u), _ptr(out), segs_dev.data_ptr(), len(layout.names), layout.total, mode, levels,
        beta, gamma, momentum, threshold, scale, channel.hist.data_ptr(), channel.sparse_state.data_ptr(),
        channel.barrier.data_ptr(), channel.status.data_ptr(), cap, phases, heap.rank, heap.world, seq,
        channel.timeout_ns, heap.bases, channel.ready_off, channel.ack_off, channel.slot_off[seq & 1], grid,
        _stream_ptr(channel.device.index), channel.cand.data_ptr() if cand_cap else 0,
        (channel.cand.data_ptr() + 4 * cand_cap) if cand_cap else 0, cand_cap,
        _ptr(kprefix), _ptr(seg_seed), rk_step & 0xFFFFFFFF,
        channel.clip_off if clip else 0, channel.clip_ready_off if clip else 0,
        channel.clip_sq.data_ptr() if clip else 0, int(strict), GRAD_DTYPE[g.dtype],
        td[0].data_ptr() if td else 0, td[1].data_ptr() if td else 0, td[2].data_ptr() if td else 0,
        channel.slot_bytes, 1 if len(layout.names) == channel._hist_segs else 0,   # hinted histograms: the layout the areas were sized for
    )
    channel.post_status()
    return seq


def run_quant(channel: ExchangeChannel, layout: FlatLayout, segs_dev: torch.Tensor, g: torch.Tensor,
              acc: Optional[torch.Tensor], mom: Optional[torch.Tensor], out: Optional[torch.Tensor], *, codec: int,
              quantum: int = 0, deterministic: bool = False, first_step: bool = False, beta: float = 1.0,
              gamma: float = 1.0, mom_beta: float = 0.0, lr: float = 1.0, scale: float = 1.0, seed: int = 0,
              step: int = 0, phases: int = PHASE_ALL, seq: Optional[int] = None, grid: Optional[int] = None,
              alltoall: bool = False, recv=None, qsgd_bucket: int = 0, qsgd_nbuckets: int = 0,
              slot_bytes: Optional[int] = None, pipeline: Optional[Tuple[int, int, int]] = None) -> int:
    """``recv``: ``(NvlsBuffer, stride)`` of the push transport (two parities of ``world`` regions of ``stride``
    bytes each), or None for the pull transport.  ``pipeline``: ``(chunks, tiles per chunk, elements per tile)`` from
    ``pipeline_plan`` runs the pipelined kernel (whole exchange in one launch, pull transport only)."""
    C = native()
    heap = channel.heap
    if seq is None:
        seq = channel.next_seq()
    if grid is None:
        grid = channel.max_grid("quant")
    need = -(-layout.total // 2048)
    grid = max(1, min(grid, max(need, 1)))
    for t in (acc, mom):
        if t is not None:
            assert t.dtype == torch.float32 and t.is_cuda and t.data_ptr() % 16 == 0, "fp32, cuda, 16-byte aligned"
    assert g.is_cuda and g.dtype in GRAD_DTYPE and g.data_ptr() % (16 if g.dtype == torch.float32 else 8) == 0, \
        "gradients: fp32 (16-byte aligned), bf16 or fp16 (8-byte aligned) on the GPU"
    assert out is None or (out.dtype == g.dtype and out.data_ptr() % (16 if g.dtype == torch.float32 else 8) == 0), \
        "the output has the gradient's element type"
    recv_local = recv_mc = recv_stride = 0
    if recv is not None and phases == PHASE_ALL:
        buf, recv_stride = recv
        parity_off = (seq & 1) * heap.world * recv_stride
        recv_local, recv_mc = buf.base_ptr + parity_off, buf.multicast_ptr + parity_off
    C.quant_exchange(
        _ptr(g), _ptr(acc), _ptr(mom), _ptr(out), segs_dev.data_ptr(), len(layout.names), layout.total, codec, quantum,
        int(deterministic), int(first_step), beta, gamma, mom_beta, lr, scale, seed & (2 ** 64 - 1), step & 0xFFFFFFFF,
        channel.quant_stats.data_ptr(), channel.barrier.data_ptr(), channel.status.data_ptr(), phases, heap.rank,
        heap.world, seq, channel.timeout_ns, heap.bases, channel.ready_off, channel.ack_off, channel.slot_off[seq & 1],
        grid, _stream_ptr(channel.device.index), int(alltoall), channel.ready2_off, recv_local, recv_mc, recv_stride, GRAD_DTYPE[g.dtype],
        int(qsgd_bucket), int(qsgd_nbuckets), channel.slot_bytes if slot_bytes is None else int(slot_bytes),
        channel.pipe.data_ptr() if pipeline else 0, channel.chunk_ready_off if pipeline else 0,
        *(pipeline if pipeline else (0, 0, 0)),
    )
    channel.post_status()
    return seq


def pipeline_plan(total: int, world: int, codec: int, force: bool = False) -> Optional[Tuple[int, int, int]]:
    """(chunks, tiles per chunk, elements per tile) of the pipelined quantised exchange, or None where it does not
    apply: QSGD with 128-element buckets and natural compression, 2..8 ranks, at least two chunks of 16 Mi elements
    (smaller exchanges are dominated by the fixed cost of a launch, not by the order of their phases).  ``force``
    drops the size and rank-count limits (tests)."""
    if codec not in (CODEC["qsgd"], CODEC["natural"]) or world > 8:
        return None
    if not force and (world < 2 or total < (32 << 20)):
        return None
    item = 65536 if total >= (128 << 20) else (32768 if total >= (64 << 20) else (16384 if total >= (1 << 20) else 8192))
    items = -(-total // item)
    chunks = max(1, min(native().PIPE_MAX_CHUNKS, total // (16 << 20) if not force else 4, items))
    per_chunk = -(-items // chunks)
    chunks = -(-items // per_chunk)
    return chunks, per_chunk, item


def segments_to_device(layout: FlatLayout, ks: Optional[Sequence[int]], device) -> torch.Tensor:
    raw = np.frombuffer(layout.segment_bytes(ks), dtype=np.uint8).copy()
    return torch.from_numpy(raw).to(device)
