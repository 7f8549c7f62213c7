"""Stand-alone quantisation ops on CUDA tensors.

Each runs the compress phase of ``csrc/quant_exchange.cu`` on a single-rank
heap and returns reference-shaped payloads (one code per element), so that
``compressor.compress()`` on a CUDA tensor uses the same encoder as the fused
exchange.  Random draws come from Philox4x32-10 keyed by (seed, name) with the
per-name call count as the step (see ``utils/philox.py``).
"""
from __future__ import annotations

import zlib
from typing import Dict, Tuple

import torch

from . import native
from .exchange import CODEC, PHASE_COMPRESS, ExchangeChannel, FlatLayout, run_quant, segments_to_device
from ..parallel.symm import SymmetricHeap

_steps: Dict[str, int] = {}
GLOBAL_SEED = 0


def _seed_step(name: str) -> Tuple[int, int]:
    step = _steps.get(name, 0)
    _steps[name] = step + 1
    return ((GLOBAL_SEED & 0xFFFFFFFF) << 32) | (zlib.crc32(name.encode("utf8")) & 0xFFFFFFFF), step


def _prep(flat: torch.Tensor) -> torch.Tensor:
    if flat.dtype != torch.float32 or not flat.is_contiguous() or flat.data_ptr() % 16 != 0:
        flat = flat.float().contiguous().clone()
    return flat


def _compress(flat, codec, name, **kw):
    C = native()
    x = _prep(flat)
    layout = FlatLayout.single(name, x.numel())
    slot_bytes = C.quant_slot_bytes(codec, layout.total, 1)
    heap = SymmetricHeap.local(2 * ((slot_bytes + 255) // 256 * 256) + 1024, x.device)
    ch = ExchangeChannel(heap, slot_bytes, 1)
    segs = segments_to_device(layout, None, x.device)
    if "seed" not in kw:
        kw["seed"], kw["step"] = _seed_step(name)
    seq = run_quant(ch, layout, segs, x, None, None, None, codec=codec, beta=0.0, gamma=1.0, phases=PHASE_COMPRESS, **kw)
    return ch, seq, layout


HEADER = 128


def _codes_offset(nseg: int) -> int:
    return HEADER + (nseg * 16 + 127) // 128 * 128


def qsgd_compress(flat, quantum_num, bucket_size, name, **kw):
    if bucket_size != 128 or quantum_num >= 128:
        raise NotImplementedError("the CUDA QSGD encoder handles bucket_size=128 and quantum_num<128")
    ch, seq, layout = _compress(flat, CODEC["qsgd"], name, quantum=int(quantum_num), **kw)
    n = flat.numel()
    off = _codes_offset(1)
    codes = ch.slot_view(seq, n, torch.int8, off).clone()
    norms = ch.slot_view(seq, layout.total // 128, torch.float32, off + layout.total).clone()
    return codes, norms


def natural_compress(flat, name, deterministic=False, **kw):
    ch, seq, layout = _compress(flat, CODEC["natural"], name, deterministic=deterministic, **kw)
    return ch.slot_view(seq, flat.numel(), torch.uint8, _codes_offset(1)).clone()


def unpack_bits(words: torch.Tensor, planes: int, numel: int) -> torch.Tensor:
    """Undo the ballot packing: ``words`` is int32 ``[groups, planes*4]``; plane
    ``q`` word ``j`` bit ``l`` belongs to element ``128*group + 4*l + j``.
    Returns uint8 ``[planes, numel]``."""
    g = words.shape[0]
    w = words.view(g, planes, 4, 1).to(torch.int64) & 0xFFFFFFFF
    lanes = torch.arange(32, device=words.device).view(1, 1, 1, 32)
    bits = (w >> lanes) & 1                      # [g, planes, j, l]
    bits = bits.permute(1, 0, 3, 2).reshape(planes, g * 128)
    return bits[:, :numel].to(torch.uint8)


def terngrad_compress(flat, name, **kw):
    ch, seq, layout = _compress(flat, CODEC["terngrad"], name, **kw)
    groups = layout.total // 128
    words = ch.slot_view(seq, groups * 8, torch.int32, _codes_offset(1)).view(groups, 8)
    planes = unpack_bits(words, 2, flat.numel())
    tern = planes[0].to(torch.int8) * (1 - 2 * planes[1].to(torch.int8))
    scale = ch.slot_view(seq, 4, torch.float32, HEADER)[:1].clone()
    return tern, scale
