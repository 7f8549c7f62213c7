"""Horovod-flavoured helper API over ``torch.distributed``.

Scripts written for the reference's Horovod integration call a handful of
``hvd.*`` functions besides ``DistributedOptimizer``
(``patch_files/horovod/torch/mpi_ops.py``: ``size``, ``rank``, ``allreduce_async_``,
``allgather_async``, ``broadcast_async``, ``synchronize``, ``poll``;
``examples/torch/pytorch_mnist.py:106-107``: ``broadcast_parameters``,
``broadcast_optimizer_state``).  This module offers the same names on top of
the process group, so such scripts only change their import:

    import grace_b200.parallel.hvd as hvd
    hvd.init(); hvd.broadcast_parameters(model.state_dict(), root_rank=0)
    optimizer = hvd.DistributedOptimizer(optimizer, grace=grc, named_parameters=model.named_parameters())
"""
from __future__ import annotations

import os
from typing import Any, Dict, Iterable, Optional, Tuple, Union

import torch
import torch.distributed as dist

from .optimizer import Average, DistributedOptimizer, Sum  # noqa: F401
from ..utils.timeline import start_timeline, stop_timeline  # noqa: F401  (same names as horovod.torch)

_handles: Dict[int, Tuple[Any, torch.Tensor, Optional[float]]] = {}
_next_handle = 0


def init(backend: Optional[str] = None) -> None:
    """Join the process group described by RANK / WORLD_SIZE / MASTER_* (no-op when already initialised)."""
    if dist.is_initialized():
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group(backend, rank=int(os.environ.get("RANK", "0")),
                            world_size=int(os.environ.get("WORLD_SIZE", "1")))
    if backend == "nccl":
        torch.cuda.set_device(local_rank())


def shutdown() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def _register(work, tensor, scale=None) -> int:
    global _next_handle
    _next_handle += 1
    _handles[_next_handle] = (work, tensor, scale)
    return _next_handle


def allreduce_async_(tensor: torch.Tensor, average: bool = True, name: Optional[str] = None, op=None) -> int:
    """In-place all-reduce; returns a handle for ``synchronize``."""
    if op is not None:
        average = op == Average
    work = dist.all_reduce(tensor, async_op=True) if size() > 1 else None
    return _register(work, tensor, 1.0 / size() if average else None)


def allreduce_(tensor: torch.Tensor, average: bool = True, name: Optional[str] = None) -> torch.Tensor:
    return synchronize(allreduce_async_(tensor, average, name))


def allreduce(tensor: torch.Tensor, average: bool = True, name: Optional[str] = None) -> torch.Tensor:
    return allreduce_(tensor.clone(), average, name)


def allgather_async(tensor: torch.Tensor, name: Optional[str] = None) -> int:
    """Concatenate along dim 0 (first dimensions may differ between ranks, as in Horovod)."""
    if size() == 1:
        return _register(None, tensor.clone())
    n = torch.tensor([tensor.shape[0]], dtype=torch.int64, device=tensor.device)
    sizes = [torch.empty_like(n) for _ in range(size())]
    dist.all_gather(sizes, n)
    sizes = [int(s) for s in sizes]
    widest = max(sizes)
    padded = tensor.new_zeros((widest,) + tuple(tensor.shape[1:]))
    padded[: tensor.shape[0]] = tensor
    outs = [torch.empty_like(padded) for _ in range(size())]
    work = dist.all_gather(outs, padded, async_op=True)
    return _register((work, outs, sizes), tensor)


def allgather(tensor: torch.Tensor, name: Optional[str] = None) -> torch.Tensor:
    return synchronize(allgather_async(tensor, name))


def broadcast_async_(tensor: torch.Tensor, root_rank: int, name: Optional[str] = None) -> int:
    work = dist.broadcast(tensor, root_rank, async_op=True) if size() > 1 else None
    return _register(work, tensor)


broadcast_async = broadcast_async_


def broadcast_(tensor: torch.Tensor, root_rank: int, name: Optional[str] = None) -> torch.Tensor:
    return synchronize(broadcast_async_(tensor, root_rank, name))


def poll(handle: int) -> bool:
    work = _handles[handle][0]
    if isinstance(work, tuple):
        work = work[0]
    return True if work is None else work.is_completed()


def synchronize(handle: int) -> torch.Tensor:
    work, tensor, scale = _handles.pop(handle)
    if isinstance(work, tuple):  # all-gather
        w, outs, sizes = work
        w.wait()
        return torch.cat([o[:n] for o, n in zip(outs, sizes)], dim=0)
    if work is not None:
        work.wait()
    if scale is not None:
        tensor.mul_(scale) if tensor.is_floating_point() else None
    return tensor


def broadcast_parameters(params: Union[Dict[str, torch.Tensor], Iterable[Tuple[str, torch.Tensor]]], root_rank: int = 0) -> None:
    """Make every replica start from rank ``root_rank``'s values (model.state_dict() or named_parameters())."""
    items = params.items() if isinstance(params, dict) else params
    handles = [broadcast_async_(t.data if hasattr(t, "data") else t, root_rank) for _, t in items if torch.is_tensor(t)]
    for h in handles:
        synchronize(h)


def broadcast_optimizer_state(optimizer: torch.optim.Optimizer, root_rank: int = 0) -> None:
    """Broadcast hyper-parameters and per-parameter state tensors of ``optimizer``."""
    if size() == 1:
        return
    payload = [optimizer.state_dict() if rank() == root_rank else None]
    dist.broadcast_object_list(payload, src=root_rank)
    if rank() != root_rank:
        optimizer.load_state_dict(payload[0])


# ---------------------------------------------------------------------------
# Smaller pieces of the Horovod surface that training scripts use
# (patch_files/horovod/torch/__init__.py:26-50, mpi_ops.py:846-861, compression.py)
# ---------------------------------------------------------------------------
def is_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def local_size() -> int:
    """Ranks on this node (torchrun's LOCAL_WORLD_SIZE; the whole job when it is not set)."""
    return int(os.environ.get("LOCAL_WORLD_SIZE", size()))


def cross_rank() -> int:
    """Index of this node among the nodes of the job."""
    return rank() // max(local_size(), 1)


def cross_size() -> int:
    return max(size() // max(local_size(), 1), 1)


def barrier() -> None:
    if size() > 1:
        dist.barrier()


def join() -> int:
    """Horovod's ``join``: block until every rank has called it; returns the rank that arrived last.

    Ranks publish their arrival time through an all-gather, so the answer is the same everywhere."""
    if size() == 1:
        return 0
    import time

    stamp = torch.tensor([time.time()], dtype=torch.float64)
    if dist.get_backend() == "nccl":
        stamp = stamp.cuda()
    stamps = [torch.zeros_like(stamp) for _ in range(size())]
    dist.all_gather(stamps, stamp)
    return int(torch.stack([s.cpu() for s in stamps]).flatten().argmax())


def broadcast_object(obj: Any, root_rank: int = 0, name: Optional[str] = None) -> Any:
    if size() == 1:
        return obj
    box = [obj if rank() == root_rank else None]
    dist.broadcast_object_list(box, src=root_rank)
    return box[0]


def allgather_object(obj: Any, name: Optional[str] = None) -> list:
    if size() == 1:
        return [obj]
    out = [None] * size()
    dist.all_gather_object(out, obj)
    return out


def metric_average(value: float, name: Optional[str] = None) -> float:
    """Average a Python number over the ranks (the reference's example averages its test metrics this way,
    ``examples/torch/pytorch_mnist.py:139-171``)."""
    t = torch.tensor([float(value)], dtype=torch.float64)
    if is_initialized() and dist.get_backend() == "nccl":
        t = t.cuda()
    return float(allreduce(t, average=True, name=name).cpu())


class _NoneCompressor:
    """Horovod's wire-format "compression" (not GRACE's): identity."""

    @staticmethod
    def compress(tensor):
        return tensor, None

    @staticmethod
    def decompress(tensor, ctx):
        return tensor


class _FP16Compressor:
    """Cast floating tensors to fp16 for the wire, back to their dtype afterwards."""

    @staticmethod
    def compress(tensor):
        if tensor.dtype.is_floating_point and tensor.dtype != torch.float16:
            return tensor.to(torch.float16), tensor.dtype
        return tensor, None

    @staticmethod
    def decompress(tensor, ctx):
        return tensor.to(ctx) if ctx is not None else tensor


class Compression:
    """``hvd.Compression.none`` / ``hvd.Compression.fp16`` as accepted by ``DistributedOptimizer(compression=...)``;
    only consulted for gradients that bypass ``grace`` (``num_groups > 0`` or ``op != Average``)."""

    none = _NoneCompressor
    fp16 = _FP16Compressor
