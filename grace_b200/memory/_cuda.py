"""Glue between the memory classes and the stand-alone CUDA kernels of ``ops/memory.py``."""
import torch


def state_like(state: torch.Tensor, tensor: torch.Tensor):
    """``state`` if the kernels can read it next to ``tensor`` (fp32, dense, same size and device), else None
    (the caller then falls back to torch ops, e.g. after a checkpoint was loaded onto another device)."""
    if (state is not None and state.is_cuda and state.device == tensor.device and state.dtype == torch.float32
            and state.is_contiguous() and state.numel() == tensor.numel()):
        return state
    return None


def sparse_payload(compressor, payload):
    """The index tensor of a (values, indices) payload of TopK / Threshold / DGC, else None."""
    from .. import compressor as C

    if isinstance(compressor, (C.TopKCompressor, C.ThresholdCompressor, C.DgcCompressor)) and len(payload) == 2:
        values, indices = payload
        if indices.dtype in (torch.int32, torch.int64) and indices.numel() == values.numel():
            return indices.contiguous()
    return None
