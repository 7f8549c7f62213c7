"""Core abstractions: ``Memory``, ``Compressor`` and ``Communicator``.

The three classes carry the whole public contract of the framework:

* a ``Memory`` keeps the error-feedback state of every named gradient
  (``compensate`` before compression, ``update`` after it);
* a ``Compressor`` turns a dense gradient into a list of payload tensors plus a
  rank-local context, and back (``compress`` / ``decompress`` / ``aggregate``);
* a ``Communicator`` owns one of each and moves payloads between ranks.

Two call styles are offered by the same ``Communicator`` object:

* ``step(tensor, name)``: blocking, returns the aggregated gradient.  Mirrors
  the contract of ``grace_dl/dist/__init__.py:37-51`` of the reference
  (compensate -> compress -> memory.update -> send_receive).
* ``send_step(tensor, name)`` / ``receive_step(handles, ctx)``: split-phase so a
  backward hook can launch the exchange and ``optimizer.step()`` can collect it
  later.  Mirrors ``grace_dl/torch/__init__.py:37-58`` of the reference.

Unlike the reference, all state that must survive a restart is reachable through
``state_dict()`` / ``load_state_dict()`` on every class.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, List, Sequence, Tuple

import torch


def _clone_tensor_dict(d: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.detach().clone() for k, v in d.items()}


class Memory(ABC):
    """Error-feedback memory.  Reference: ``grace_dl/dist/__init__.py:4-12``."""

    #: names of dict attributes (name -> tensor) that make up the checkpoint state
    _state_fields: Tuple[str, ...] = ()

    @abstractmethod
    def compensate(self, tensor: torch.Tensor, name: str) -> torch.Tensor:
        """Return the tensor that should be compressed (gradient + feedback)."""

    def update(self, tensor, name, compressor, tensor_compressed, ctx) -> None:
        """Record what compression lost.  Default: stateless."""
        return None

    # -- checkpoint -------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        return {f: _clone_tensor_dict(getattr(self, f)) for f in self._state_fields}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        for f in self._state_fields:
            if f in state:
                target = getattr(self, f)
                target.clear()
                target.update(_clone_tensor_dict(state[f]))


class Compressor(ABC):
    """Lossy codec for one gradient tensor.

    ``average``: divide the aggregate by the world size.
    ``tensors_size_are_same``: every rank's payload has the same shape, so the
    communicator may skip the size exchange.
    Reference: ``grace_dl/dist/__init__.py:15-34``.
    """

    _state_fields: Tuple[str, ...] = ()

    def __init__(self, average: bool = True, tensors_size_are_same: bool = True):
        self.average = average
        self.tensors_size_are_same = tensors_size_are_same

    @abstractmethod
    def compress(self, tensor: torch.Tensor, name: str) -> Tuple[Sequence[torch.Tensor], Any]:
        """Return ``(payload_tensors, ctx)``.  Only the payload crosses ranks."""

    @abstractmethod
    def decompress(self, tensors: Sequence[torch.Tensor], ctx: Any) -> torch.Tensor:
        """Rebuild a dense tensor from one rank's payload."""

    def aggregate(self, tensors: List[torch.Tensor]) -> torch.Tensor:
        """Combine the W decompressed tensors.  Default: element-wise sum."""
        out = tensors[0].clone()
        for t in tensors[1:]:
            out += t
        return out

    # -- checkpoint -------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for f in self._state_fields:
            v = getattr(self, f)
            out[f] = _clone_tensor_dict(v) if isinstance(v, dict) else v
        return out

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        for f in self._state_fields:
            if f not in state:
                continue
            cur = getattr(self, f)
            if isinstance(cur, dict):
                cur.clear()
                cur.update(_clone_tensor_dict(state[f]))
            else:
                setattr(self, f, state[f])


class Communicator(ABC):
    """Owns a compressor and a memory and performs the exchange.

    Sub-classes implement either ``send_receive`` (blocking) or the pair
    ``async_send`` / ``wait_receive``; each default is written in terms of the
    other so that both call styles work on every communicator.
    """

    def __init__(self, compressor: Compressor, memory: Memory, world_size: int = 1):
        self.compressor = compressor
        self.memory = memory
        self.world_size = int(world_size)
        self._stats: Dict[str, float] = {"steps": 0, "payload_bytes": 0, "dense_bytes": 0}

    # -- blocking style ---------------------------------------------------
    def send_receive(self, tensors, name, ctx) -> torch.Tensor:
        handles = self.async_send(tensors, name)
        return self.wait_receive(handles, ctx)

    def step(self, tensor: torch.Tensor, name: str) -> torch.Tensor:
        from .utils import timeline

        tl = timeline.active()
        tok = tl.begin(name, type(self).__name__, device=tensor.is_cuda, numel=tensor.numel(),
                       compressor=type(self.compressor).__name__) if tl is not None else None
        tensor = self.memory.compensate(tensor, name)
        payload, ctx = self.compressor.compress(tensor, name)
        self.memory.update(tensor, name, self.compressor, payload, ctx)
        self._account(tensor, payload)
        out = self.send_receive(payload, name, ctx)
        if tok is not None:
            tl.end(tok, payload_bytes=sum(t.numel() * t.element_size() for t in payload))
        return out

    # -- split-phase style ------------------------------------------------
    def async_send(self, tensors, name):
        raise NotImplementedError("async_send or send_receive must be implemented")

    def wait_receive(self, handles, ctx) -> torch.Tensor:
        raise NotImplementedError("wait_receive or send_receive must be implemented")

    def send_step(self, tensor: torch.Tensor, name: str):
        tensor = self.memory.compensate(tensor, name)
        payload, ctx = self.compressor.compress(tensor, name)
        self.memory.update(tensor, name, self.compressor, payload, ctx)
        self._account(tensor, payload)
        handles = self.async_send(payload, name)
        return handles, ctx

    def receive_step(self, handles, ctx) -> torch.Tensor:
        return self.wait_receive(handles, ctx)

    # -- observability ----------------------------------------------------
    def _account(self, tensor: torch.Tensor, payload) -> None:
        self._stats["steps"] += 1
        self._stats["dense_bytes"] += tensor.numel() * tensor.element_size()
        self._stats["payload_bytes"] += sum(t.numel() * t.element_size() for t in payload)

    def stats(self) -> Dict[str, float]:
        """Counters since construction: steps, payload bytes, achieved ratio."""
        s = dict(self._stats)
        s["compression_ratio"] = (s["dense_bytes"] / s["payload_bytes"]) if s["payload_bytes"] else float("inf")
        return s

    # -- checkpoint -------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        return {
            "compressor": self.compressor.state_dict(),
            "memory": self.memory.state_dict(),
            "world_size": self.world_size,
        }

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self.compressor.load_state_dict(state.get("compressor", {}))
        if state.get("world_size", self.world_size) != self.world_size:
            import warnings

            warnings.warn(
                "grace checkpoint was written with world_size=%s, now %s: "
                "error-feedback state is per-rank and is reset to zero"
                % (state.get("world_size"), self.world_size)
            )
            return
        self.memory.load_state_dict(state.get("memory", {}))
