"""Stand-alone sparse ops on CUDA tensors: exact top-k selection by magnitude.

Runs the compress phase of ``csrc/sparse_exchange.cu`` on a single-rank heap:
histogram, on-device radix select of the k-th magnitude, compaction.  No host
synchronisation, no sort.  Replaces ``torch.topk`` / the reference's
``rdxtopk`` extension (``radixtopk_cuda/rdxtopk_cuda.cu``).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import native
from .exchange import (PHASE_COMPRESS, SPARSE_TOPK, ExchangeChannel, FlatLayout, run_sparse, segments_to_device)
from ..parallel.symm import SymmetricHeap


def topk_select(flat: torch.Tensor, k: int, exact: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Values (signed, fp32) and int32 indices of the k largest |x|; unsorted.

    Ties at the k-th magnitude are broken arbitrarily; exactly k entries are
    returned.  ``exact=False`` resolves only the top 24 key bits.
    """
    C = native()
    assert flat.is_cuda and flat.dim() == 1
    x = flat
    if x.dtype != torch.float32 or not x.is_contiguous() or x.data_ptr() % 16 != 0:
        x = x.float().contiguous().clone()
    n = x.numel()
    k = max(1, min(int(k), n))
    layout = FlatLayout.single("t", n)
    cap = (k + 15) // 16 * 16
    slot_bytes = C.sparse_slot_bytes(cap)
    heap = SymmetricHeap.local(2 * ((slot_bytes + 255) // 256 * 256) + 1024, x.device)
    ch = ExchangeChannel(heap, slot_bytes, 1)
    segs = segments_to_device(layout, [k], x.device)
    seq = run_sparse(ch, layout, segs, x, None, None, None, mode=SPARSE_TOPK, cap=cap, beta=0.0, gamma=1.0,
                     levels=3 if exact else 2, phases=PHASE_COMPRESS)
    vals = ch.slot_view(seq, k, torch.float32, 128)
    idx = ch.slot_view(seq, k, torch.int32, 128 + cap * 4)
    return vals.clone(), idx.clone()
