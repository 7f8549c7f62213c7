"""``rdxtopk.topk(input, indices, k)`` with the call signature of the reference's radix-select extension
(``grace_dl/dist/compressor/radixtopk_cuda/rdxtopk.cpp:1-18``; used by ``topk.py:7-15`` as
``vals, idx = rdxtopk.topk(tensor.abs(), arange, k)``).

Returns the k largest values of ``input`` (unsorted) and the entries of ``indices`` at their positions, as
``(float32[k], int32[k])``.  CUDA tensors with no negative entry - the only way the reference calls it - use this
package's on-device radix select (``grace_b200.ops.sparse.topk_select``: no host round trip per digit, no
allocation per call); everything else goes through ``torch.topk``.
"""
import torch


def topk(input: torch.Tensor, indices: torch.Tensor, k: int):
    flat = input.reshape(-1)
    k = int(k)
    if flat.is_cuda and flat.dtype == torch.float32 and 0 < k <= flat.numel() and bool((flat >= 0).all()):
        from grace_b200.ops.sparse import topk_select

        vals, pos = topk_select(flat.contiguous(), k)
        pos = pos.long()
    else:
        vals, pos = torch.topk(flat, k, sorted=False)
    picked = indices.reshape(-1)[pos] if indices is not None else pos
    return vals.float(), picked.int()
