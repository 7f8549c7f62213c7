"""Thin helpers over ``torch.distributed`` used by the library-call
communicators (the baseline paths)."""
from __future__ import annotations

from typing import List

import torch
from torch import distributed as dist


def active() -> bool:
    return dist.is_available() and dist.is_initialized()


def backend_supports_all_to_all() -> bool:
    return active() and dist.get_backend() in ("nccl", "mpi")


def all_to_all(outputs: List[torch.Tensor], inputs: List[torch.Tensor]) -> None:
    """``dist.all_to_all`` with a gather-based stand-in for backends that lack
    it (gloo), so the two-phase protocol can be tested on CPU ranks."""
    if backend_supports_all_to_all():
        dist.all_to_all(outputs, inputs)
        return
    world = dist.get_world_size()
    rank = dist.get_rank()
    stacked = torch.stack([t.contiguous() for t in inputs])
    gathered = [torch.empty_like(stacked) for _ in range(world)]
    dist.all_gather(gathered, stacked)
    for src in range(world):
        outputs[src].copy_(gathered[src][rank])
