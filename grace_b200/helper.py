"""``grace_from_params(dict) -> Communicator``.

Keys, defaults and accepted names follow ``grace_dl/dist/helper.py:1-102`` and
``grace_dl/torch/helper.py:1-91`` of the reference, plus the TensorFlow-only
codecs of ``grace_dl/tensorflow/helper.py`` (``adaq``, ``inceptionn``,
``sketch``, ``u8bit``).  Additional optional keys:

``fused`` (bool, default False)
    use the single-kernel sm_100a exchange (``communicator/fused.py``) instead
    of the ``torch.distributed`` communicators when the combination supports it.
``compress_rank`` / ``rank`` (PowerSGD)
    reaches both the compressor and the memory (the reference only forwards it
    to the memory).
``seed``, ``timeout_ms``, ``comm_sms``
    forwarded to the fused exchange.
``deterministic`` (natural compression, default False)
    round to the nearest power of two instead of drawing (the reference's
    ``cnat_cuda.compress_deterministic``, which its helper never reaches).
``nvls`` / ``use_nvls`` (bool, default False; needs ``fused``)
    use the NVSwitch multicast mapping where it is available and the job has
    at least ``nvls_min_world`` (default 4) ranks: the ``none`` compressor with
    no memory averages with ``multimem.ld_reduce`` (``communicator/nvls.py``);
    the quantised codecs in all-gather mode push their encoded slots to every
    GPU with ``multimem.st`` and decode from local memory.  The peer-load
    exchange stays the fallback.

Unknown names raise ``NotImplementedError`` as in the reference.
"""
from __future__ import annotations

from typing import Any, Callable, Dict

from . import compressor as C
from . import memory as M
from . import communicator as K


def _world(params):
    if "world_size" in params:
        return params["world_size"]
    from torch import distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size()
    raise KeyError("world_size")


_COMPRESSORS: Dict[str, Callable[[Dict[str, Any]], Any]] = {
    "none": lambda p: C.NoneCompressor(),
    "fp16": lambda p: C.FP16Compressor(),
    "topk": lambda p: C.TopKCompressor(p.get("compress_ratio", 0.3), p.get("kernel", "torch")),
    "randomk": lambda p: C.RandomKCompressor(p.get("compress_ratio", 0.3)),
    "threshold": lambda p: C.ThresholdCompressor(p.get("threshold", 0.01)),
    "dgc": lambda p: C.DgcCompressor(p.get("compress_ratio", 0.3)),
    "qsgd": lambda p: C.QSGDCompressor(p.get("quantum_num", 127), p.get("bucket_size", 128)),
    "qsgd_cuda": lambda p: C.QSGDCompressor_CUDA(p.get("quantum_num", 127), p.get("bucket_size", 128)),
    "terngrad": lambda p: C.TernGradCompressor(),
    "signsgd": lambda p: C.SignSGDCompressor(),
    "signum": lambda p: C.SignumCompressor(p.get("momentum", 0.9)),
    "efsignsgd": lambda p: C.EFSignSGDCompressor(p.get("lr", 0.1)),
    "onebit": lambda p: C.OneBitCompressor(),
    "natural": lambda p: C.NaturalCompressor(deterministic=bool(p.get("deterministic", False))),
    "natural_cuda": lambda p: C.NaturalCompressor_CUDA(deterministic=bool(p.get("deterministic", False))),
    "u8bit": lambda p: C.U8bitCompressor(),
    "8bit": lambda p: C.U8bitCompressor(),
    "powersgd": lambda p: C.PowerSGDCompressor(
        rank=p.get("compress_rank", p.get("rank", 1)),
        use_memory=p.get("use_memory", False),
        world_size=_world(p) if ("world_size" in p) else 1,
    ),
    "adaq": lambda p: C.AdaqCompressor(p.get("compress_ratio", 0.3)),
    "inceptionn": lambda p: C.INCEPTIONNCompressor(p.get("error_bound", 2e-10)),
    "sketch": lambda p: C.SketchCompressor(p.get("quantiles", 64)),
}

_MEMORIES: Dict[str, Callable[[Dict[str, Any], Any], Any]] = {
    "none": lambda p, comp: M.NoneMemory(),
    "residual": lambda p, comp: M.ResidualMemory(p.get("beta", 1.0), p.get("gamma", 1.0)),
    "efsignsgd": lambda p, comp: M.EFSignSGDMemory(p.get("lr", 0.1)),
    "dgc": lambda p, comp: M.DgcMemory(p.get("momentum", 0.9), p.get("gradient_clipping", False), p["world_size"]),
    "powersgd": lambda p, comp: M.PowerSGDMemory(comp.q_memory, p.get("compress_rank", p.get("rank", 1))),
}

_COMMUNICATORS: Dict[str, Callable[..., Any]] = {
    "allreduce": lambda comp, mem, p: K.Allreduce(comp, mem, _world(p)),
    "allgather": lambda comp, mem, p: K.Allgather(comp, mem, _world(p)),
    "broadcast": lambda comp, mem, p: K.Broadcast(comp, mem, _world(p), p.get("rank")),
    "alltoall": lambda comp, mem, p: K.AllToAll(comp, mem, _world(p)),
}


def _nvls(params) -> bool:
    return bool(params.get("nvls", params.get("use_nvls", False)))


def grace_from_params(params: Dict[str, Any]):
    comp_name = params.get("compressor", "none")
    mem_name = params.get("memory", "none")
    comm_name = params.get("communicator", "allreduce")
    if comp_name not in _COMPRESSORS:
        raise NotImplementedError(comp_name)
    if mem_name not in _MEMORIES:
        raise NotImplementedError(mem_name)
    if comm_name not in _COMMUNICATORS and comm_name != "fused":
        raise NotImplementedError(comm_name)
    comp = _COMPRESSORS[comp_name](params)
    mem = _MEMORIES[mem_name](params, comp)
    host = None
    if params.get("host_protocol", False):
        # CPU ranks: the fused exchange protocol over POSIX shared memory (csrc/host_exchange.cpp)
        from .communicator.host import HostExchange

        host = HostExchange(comp, mem, _world(params), world=params.get("host_world"), group=params.get("group"),
                            seed=params.get("seed", 0), timeout_ms=params.get("timeout_ms", 10000),
                            arena_mb=params.get("arena_mb", 16), store=params.get("store"),
                            mode="alltoall" if comm_name == "alltoall" else "allgather")
        if not (params.get("fused", False) or comm_name == "fused"):
            return host
    if params.get("fused", False) or comm_name == "fused":
        from .communicator.fused import FusedExchange

        mode = "alltoall" if comm_name == "alltoall" else "allgather"
        fused = FusedExchange(
            comp, mem, _world(params), mode=mode,
            seed=params.get("seed", 0), timeout_ms=params.get("timeout_ms", 10000),
            comm_sms=params.get("comm_sms"), group=params.get("group"),
            nvls=_nvls(params), nvls_min_world=params.get("nvls_min_world", 4),
            overlap_sms=params.get("overlap_sms", 32), arena_mb=params.get("arena_mb", 64),
            split_overlap=params.get("split_overlap", False), store=params.get("store"),
            pipeline=params.get("pipeline", True),
        )
        if _nvls(params) and comp_name == "none" and mem_name == "none":
            from .communicator.nvls import NvlsAllreduce

            return NvlsAllreduce(comp, mem, _world(params), fallback=fused, group=params.get("group"),
                                 timeout_ms=params.get("timeout_ms", 10000), comm_sms=params.get("comm_sms"),
                                 min_world=params.get("nvls_min_world", 4))
        if host is not None:   # both: kernels for CUDA tensors, the host engine for CPU tensors
            fused.attach_host(host)
        return fused
    return _COMMUNICATORS[comm_name](comp, mem, params)
