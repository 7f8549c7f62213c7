"""Launch plan for the fused PowerSGD exchange (``csrc/powersgd.cu``).

A ``LowRankPlan`` covers every matrix of one flat layout: tensors with at least
two dimensions whose row and column counts are multiples of four (a TMA row
stride must be a multiple of 16 bytes).  All other tensors of the layout (1-D
tensors, which PowerSGD never compresses, and oddly shaped matrices) are
exchanged densely and uncompressed by the quantised kernel's fp32 codec through
a small staging buffer.  The plan owns the tensor maps, the matrix table, the
P / Q work buffers and the persistent ``Q^T`` that warm-starts the next step.
"""
from __future__ import annotations

import struct
import zlib
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import native
from .exchange import (CODEC, PHASE_ALL, PHASE_COMPRESS, PHASE_EXCHANGE, ExchangeChannel, FlatLayout,
                       run_quant, segments_to_device, _stream_ptr)

RANK_PAD = 16
TILE_K = 32
TILE_ROWS = 128
S1_TILES = 2                  # K tiles per ring step of stage 1 (kS1Tiles of the kernel)
MIN_STEPS_PER_ITEM = 8        # a work item runs at least this many ring steps (unless the matrix is smaller)
MAX_RANK = 16


def eligible(shape: Sequence[int]) -> bool:
    if len(shape) < 2:
        return False
    n = int(shape[0])
    m = 1
    for d in shape[1:]:
        m *= int(d)
    return n % 4 == 0 and m % 4 == 0 and n >= 16 and m >= 16


def choose_splits(n_out: int, n_k: int, grid: int, tiles_per_step: int = 1) -> int:
    """K splits per 128-row block of one GEMM stage: the work items (blocks x splits) should fill whole waves of
    ``grid`` persistent CTAs, and an item should not be shorter than ``MIN_STEPS_PER_ITEM`` ring steps."""
    blocks = -(-n_out // TILE_ROWS)
    ktiles = -(-n_k // (TILE_K * tiles_per_step))      # ring steps along K
    max_splits = max(1, ktiles // MIN_STEPS_PER_ITEM)
    best, best_score = 1, -1.0
    for splits in range(1, max_splits + 1):
        items = blocks * splits
        waves = -(-items // grid)
        score = items / (waves * grid) - 1e-4 * splits     # fill of the last wave; ties go to fewer splits
        if waves * (-(-ktiles // splits)) > 0 and score > best_score + 1e-9:
            best, best_score = splits, score
    return best


def orthogonal_init(m: int, r: int, seed: int, device) -> torch.Tensor:
    """Deterministic N(0,1) start for Q (m x r), orthogonalised; identical on every rank."""
    from ..compressor.powersgd import orthogonalize

    gen = torch.Generator(device="cpu").manual_seed(seed & 0x7FFFFFFFFFFFFFFF)
    q = torch.randn(m, r, generator=gen, dtype=torch.float64)
    orthogonalize(q)
    return q.float().to(device)


class LowRankPlan:
    def __init__(self, heap_factory, layout: FlatLayout, shapes: Sequence[Sequence[int]], rank: int, world: int,
                 has_memory: bool, device, seed: int = 0, timeout_ms: float = 10000.0, sm_limit: Optional[int] = None):
        C = native()
        self.layout = layout
        self.rank = int(rank)
        self.world = world
        self.device = device
        self.has_memory = has_memory
        self.steps = 0
        if not 1 <= self.rank <= MAX_RANK:
            raise ValueError("the fused PowerSGD path supports ranks 1..%d" % MAX_RANK)
        self.matrices: List[Tuple[str, int, int, int]] = []   # name, offset, n, m
        self.others: List[int] = []                           # indices of densely exchanged tensors
        for i, (name, off, numel, shape) in enumerate(zip(layout.names, layout.offsets, layout.numels, shapes)):
            if eligible(shape):
                n = int(shape[0])
                self.matrices.append((name, off, n, numel // n))
            else:
                self.others.append(i)
        # ---- matrix table and work buffers ----
        p_off = q_off = pt_off = qt_off = 0
        i1 = i2 = 0
        rows = []
        grid = 148
        try:
            if torch.device(device).type == "cuda":
                grid = max(1, C.lowrank_max_grid(torch.device(device).index or 0, sm_limit or 0))
        except Exception:
            pass
        for name, off, n, m in self.matrices:
            s1, s2 = choose_splits(n, m, grid, S1_TILES), choose_splits(m, n, grid)
            rows.append(struct.pack("<qiiiiiiiiii", off, n, m, p_off, q_off, pt_off, qt_off, i1, i2, s1, s2))
            p_off += n * RANK_PAD
            q_off += m * RANK_PAD
            pt_off += n * RANK_PAD
            qt_off += m * RANK_PAD
            i1 += -(-n // TILE_ROWS) * s1
            i2 += -(-m // TILE_ROWS) * s2
        self.p_floats, self.q_floats = p_off, q_off
        self.items_s1, self.items_s2 = i1, i2
        nmat = len(self.matrices)
        self.acc = torch.zeros(layout.total, dtype=torch.float32, device=device) if has_memory else None
        if nmat:
            assert C.LOWRANK_MATRIX_BYTES == len(rows[0]), (C.LOWRANK_MATRIX_BYTES, len(rows[0]))
            self.mats = torch.from_numpy(np.frombuffer(b"".join(rows), dtype=np.uint8).copy()).to(device)
            self.p_mean = torch.zeros(self.p_floats, dtype=torch.float32, device=device)
            self.q_mean = torch.zeros(self.q_floats, dtype=torch.float32, device=device)
            self.pt_orth = torch.zeros(self.p_floats, dtype=torch.float32, device=device)
            self.qt = torch.zeros(self.q_floats, dtype=torch.float32, device=device)
            self.gram = torch.zeros(max(grid, 160) * nmat * 256, dtype=torch.float64, device=device)   # per-CTA partials
            # split-K scratch: one 128 x 16 block of partial sums per work item
            self.partial = torch.empty((self.items_s1 + self.items_s2) * TILE_ROWS * RANK_PAD, dtype=torch.float32,
                                       device=device)
            qt_off = 0
            for name, off, n, m in self.matrices:
                r = min(n, m, self.rank)
                q0 = orthogonal_init(m, r, seed ^ zlib.crc32(name.encode('utf8')), device)
                self.qt[qt_off : qt_off + r * m].view(r, m).copy_(q0.t())
                qt_off += m * RANK_PAD
            slot_bytes = (self.p_floats + self.q_floats) * 4
            self.heap = heap_factory(("lowrank",) + layout.key(), 2 * ((slot_bytes + 255) // 256 * 256) + 8192)
            self.channel = ExchangeChannel(self.heap, slot_bytes, 1, timeout_ms, sm_limit)
            self.ready2_off = self.channel.ready2_off or self.heap.alloc(C.MAX_WORLD * 8)
            self.maps = None
            self._maps_key = None
        # ---- dense side channel for everything that is not a matrix ----
        self.dense = None
        if self.others:
            names = [layout.names[i] for i in self.others]
            numels = [layout.numels[i] for i in self.others]
            self.dense_layout = FlatLayout(names, numels)
            idx = []
            for i, o2 in zip(self.others, self.dense_layout.offsets):
                idx.append(torch.arange(layout.numels[i], dtype=torch.int64) + layout.offsets[i])
            self.dense_src = torch.cat(idx).to(device)
            dst = []
            for i, o2 in zip(self.others, self.dense_layout.offsets):
                dst.append(torch.arange(layout.numels[i], dtype=torch.int64) + o2)
            self.dense_dst = torch.cat(dst).to(device)
            self.dense_stage = torch.zeros(self.dense_layout.total, dtype=torch.float32, device=device)
            slot = C.quant_slot_bytes(CODEC["fp32"], self.dense_layout.total, len(names))
            self.dense_heap = heap_factory(("lowrank-dense",) + layout.key(), 2 * ((slot + 255) // 256 * 256) + 4096)
            self.dense_channel = ExchangeChannel(self.dense_heap, slot, len(names), timeout_ms, sm_limit)
            self.dense_segs = segments_to_device(self.dense_layout, None, device)
            self.dense = True

    # ------------------------------------------------------------------
    def _ensure_maps(self, g: torch.Tensor):
        C = native()
        key = (g.data_ptr(), self.acc.data_ptr() if self.acc is not None else 0)
        if self._maps_key == key:
            return
        nmat = len(self.matrices)
        nbytes = nmat * C.MAPS_PER_MATRIX * C.TENSOR_MAP_BYTES
        raw = np.zeros(nbytes + 64, dtype=np.uint8)          # tensor maps are 64-byte aligned objects
        shift = (-raw.ctypes.data) % 64
        host = raw[shift : shift + nbytes]
        base = host.ctypes.data
        pt_off = qt_off = 0
        for i, (name, off, n, m) in enumerate(self.matrices):
            C.lowrank_encode_maps(
                base + i * C.MAPS_PER_MATRIX * C.TENSOR_MAP_BYTES, g.data_ptr() + 4 * off,
                (self.acc.data_ptr() + 4 * off) if self.acc is not None else 0,
                self.qt.data_ptr() + 4 * qt_off, self.pt_orth.data_ptr() + 4 * pt_off, n, m)
            pt_off += n * RANK_PAD
            qt_off += m * RANK_PAD
        self.maps = torch.from_numpy(host.copy()).to(self.device)
        self._maps_key = key

    def launch(self, g: torch.Tensor, out: torch.Tensor, part: int = 0, seq: Optional[int] = None,
               sm_limit: Optional[int] = None) -> int:
        """Run the low-rank exchange of all matrices (``part`` 0 = everything)."""
        C = native()
        assert g.dtype == torch.float32 and g.data_ptr() % 16 == 0
        self._ensure_maps(g)
        ch = self.channel
        if seq is None:
            seq = ch.next_seq()
        grid = C.lowrank_max_grid(ch.heap.device.index, ch.sm_limit if sm_limit is None else int(sm_limit))
        heap = ch.heap
        C.powersgd_exchange(
            g.data_ptr(), self.acc.data_ptr() if self.acc is not None else 0, out.data_ptr(), self.mats.data_ptr(),
            self.maps.data_ptr(), len(self.matrices), self.rank, int(self.has_memory), self.world, self.items_s1,
            self.items_s2, self.p_floats, self.q_floats, self.p_mean.data_ptr(), self.q_mean.data_ptr(),
            self.pt_orth.data_ptr(), self.qt.data_ptr(), self.gram.data_ptr(), self.partial.data_ptr(),
            ch.barrier.data_ptr(), ch.status.data_ptr(), self.ready2_off, part, heap.rank, heap.world, seq, ch.timeout_ns, heap.bases,
            ch.ready_off, ch.ack_off, ch.slot_off[seq & 1], grid, _stream_ptr())
        ch.post_status()
        return seq

    def launch_dense(self, g: torch.Tensor, out: torch.Tensor, phases: int = PHASE_ALL, seq: Optional[int] = None,
                     sm_limit: Optional[int] = None):
        """Uncompressed mean of the non-matrix tensors (one-shot all-gather-sum)."""
        if not self.dense:
            return None
        if phases & PHASE_COMPRESS:
            self.dense_stage.index_copy_(0, self.dense_dst, g.index_select(0, self.dense_src))
        seq = run_quant(self.dense_channel, self.dense_layout, self.dense_segs, self.dense_stage, None, None,
                        self.dense_stage, codec=CODEC["fp32"], beta=0.0, gamma=1.0, scale=1.0 / self.world,
                        phases=phases, seq=seq,
                        grid=None if sm_limit is None else self.dense_channel.max_grid("quant", sm_limit))
        if phases & PHASE_EXCHANGE:
            out.index_copy_(0, self.dense_src, self.dense_stage.index_select(0, self.dense_dst))
        return seq

    def check(self):
        if self.matrices:
            self.channel.check()
        if self.dense:
            self.dense_channel.check()

    # state for checkpoints -------------------------------------------------
    def q_memory(self):
        out, qt_off = {}, 0
        for name, off, n, m in self.matrices:
            r = min(n, m, self.rank)
            out[name] = self.qt[qt_off : qt_off + r * m].view(r, m).t().clone()
            qt_off += m * RANK_PAD
        return out

    def load_q_memory(self, q_memory):
        qt_off = 0
        for name, off, n, m in self.matrices:
            r = min(n, m, self.rank)
            if name in q_memory and tuple(q_memory[name].shape) == (m, r):
                self.qt[qt_off : qt_off + r * m].view(r, m).copy_(q_memory[name].t())
            qt_off += m * RANK_PAD
