"""Checkpoint / resume.

The reference never saves GRACE state (residuals, momenta and ``q_memory``
live in Python dicts that die with the process).  Here:

* ``grace_rank{r}.pt``: ``grc.state_dict()`` of rank ``r``.  Error-feedback
  state is different on every rank, so every rank writes its own shard.  Keys
  are the reference's attribute names (``residuals``, ``gradients``,
  ``momentums``, ``q_memory``, ``global_step``).
* ``model.pt`` / ``optimizer.pt``: written by rank 0 only (replicas are
  identical).
* ``meta.pt``: step counter, world size, RNG state.

Loading with a different world size keeps the model and optimizer and resets
the error-feedback state with a warning.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch


def save_checkpoint(directory: str, model=None, optimizer=None, grace=None, rank: int = 0, step: int = 0,
                    extra: Optional[Dict[str, Any]] = None) -> None:
    os.makedirs(directory, exist_ok=True)
    if grace is not None:
        torch.save(grace.state_dict(), os.path.join(directory, "grace_rank%d.pt" % rank))
    if rank == 0:
        if model is not None:
            torch.save(model.state_dict(), os.path.join(directory, "model.pt"))
        if optimizer is not None:
            torch.save(optimizer.state_dict(), os.path.join(directory, "optimizer.pt"))
        meta = {"step": step, "torch_rng": torch.get_rng_state(), "extra": extra or {}}
        if grace is not None:
            meta["world_size"] = grace.world_size
        torch.save(meta, os.path.join(directory, "meta.pt"))


def load_checkpoint(directory: str, model=None, optimizer=None, grace=None, rank: int = 0,
                    map_location="cpu") -> Dict[str, Any]:
    meta = torch.load(os.path.join(directory, "meta.pt"), map_location="cpu", weights_only=False)
    if model is not None:
        model.load_state_dict(torch.load(os.path.join(directory, "model.pt"), map_location=map_location))
    if optimizer is not None:
        optimizer.load_state_dict(torch.load(os.path.join(directory, "optimizer.pt"), map_location=map_location))
    if grace is not None:
        shard = os.path.join(directory, "grace_rank%d.pt" % rank)
        if os.path.exists(shard):
            grace.load_state_dict(torch.load(shard, map_location=map_location, weights_only=False))
    return meta
