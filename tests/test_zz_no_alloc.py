"""The allocation-free top-k entry point (``grace_topk_select_noalloc``).

Some users of the library cannot allocate device memory where they need a
top-k: a plug-in living inside a host application that owns the allocator, code
inside a memory-planned region that has already handed out every byte it reserved, a latency-bound
loop where ``cudaMalloc`` would stall the device.  For them the library exports
one C symbol whose scratch lives in a static device array.  This test calls it
through ``ctypes`` exactly as such a caller would (raw pointers, no Python
wrapper), twice in a row on different inputs, and checks each result against
the regular ``topk_select`` op.  It is collected last so that a failure here
never hides another test's result.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from grace_b200.ops import native

    mod = native()
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.grace_topk_select_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.grace_topk_noalloc_strerror.restype = ctypes.c_char_p
    lib.grace_topk_noalloc_strerror.argtypes = [ctypes.c_int]
    lib.grace_topk_noalloc_status.restype = ctypes.c_int
    lib.grace_topk_noalloc_status.argtypes = [ctypes.POINTER(ctypes.c_uint), ctypes.c_void_p]
    return lib


def _status(lib):
    words = (ctypes.c_uint * 4)()
    rc = lib.grace_topk_noalloc_status(words, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.grace_topk_noalloc_strerror(rc)
    return list(words)


def _call(lib, x, k):
    vals = torch.empty(k, dtype=torch.float32, device=x.device)
    idx = torch.empty(k, dtype=torch.int32, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.grace_topk_select_noalloc(x.data_ptr(), x.numel(), k, vals.data_ptr(), idx.data_ptr(), stream)
    assert rc == 0, lib.grace_topk_noalloc_strerror(rc)
    return vals, idx


def test_no_alloc_topk_matches_regular_entry_point_twice():
    from grace_b200.ops.sparse import topk_select

    lib = _lib()
    dev = torch.device("cuda")
    gen = torch.Generator(device="cpu").manual_seed(1234)
    # two calls in a row share the static work area: different sizes and k on purpose
    for n, k in ((1_000_003, 10_000), (70_001, 700), (130, 130)):
        x = (torch.randn(n, generator=gen) * 1e-3).to(dev)
        vals, idx = _call(lib, x, k)
        torch.cuda.synchronize()
        assert _status(lib) == [0, 0, 0, 0]     # the kernel ran to completion: no barrier gave up
        ref_vals, ref_idx = topk_select(x, k)
        order, ref_order = idx.long().argsort(), ref_idx.long().argsort()
        assert torch.equal(idx.long()[order], ref_idx.long()[ref_order])
        assert torch.equal(vals[order], ref_vals[ref_order])
        assert torch.equal(vals, x[idx.long()])


def test_no_alloc_topk_allocates_nothing():
    """With the outputs allocated beforehand, a call takes nothing from the device's free memory (cudaMalloc by
    anyone in the process) and does not change the caching allocator's books (an allocation through torch).  Free
    memory may grow meanwhile (heaps of earlier tests whose last reference dies late), it must not shrink."""
    import gc

    lib = _lib()
    x = torch.randn(300_000, device="cuda")
    vals = torch.empty(3000, dtype=torch.float32, device="cuda")
    idx = torch.empty(3000, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = lib.grace_topk_select_noalloc(x.data_ptr(), x.numel(), 3000, vals.data_ptr(), idx.data_ptr(), stream)
        assert rc == 0, lib.grace_topk_noalloc_strerror(rc)

    call()                      # first call on the device: address look-up, kernel image load
    _status(lib)                # and the first status read-back
    gc.collect()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    stats0 = torch.cuda.memory_stats()
    call()
    call()
    torch.cuda.synchronize()
    assert _status(lib) == [0, 0, 0, 0]
    stats1 = torch.cuda.memory_stats()
    assert torch.cuda.mem_get_info()[0] >= free0
    for key in ("allocation.all.allocated", "segment.all.allocated", "allocated_bytes.all.current",
                "reserved_bytes.all.current"):
        assert stats1[key] == stats0[key], key
    assert torch.equal(vals, x[idx.long()])


def test_no_alloc_topk_rejects_bad_sizes():
    lib = _lib()
    x = torch.randn(1024, device="cuda")
    out_v = torch.empty(8, device="cuda")
    out_i = torch.empty(8, dtype=torch.int32, device="cuda")
    too_large = lib.grace_topk_select_noalloc(x.data_ptr(), 2 ** 31, 8, out_v.data_ptr(), out_i.data_ptr(), None)
    assert too_large == -2 and b"too large" in lib.grace_topk_noalloc_strerror(too_large)
    assert lib.grace_topk_select_noalloc(x.data_ptr(), 1024, 0, out_v.data_ptr(), out_i.data_ptr(), None) == -1
    assert lib.grace_topk_select_noalloc(x.data_ptr(), 4, 8, out_v.data_ptr(), out_i.data_ptr(), None) == -1
    assert lib.grace_topk_select_noalloc(None, 1024, 8, out_v.data_ptr(), out_i.data_ptr(), None) == -1
    misaligned = lib.grace_topk_select_noalloc(x.data_ptr() + 4, 1000, 8, out_v.data_ptr(), out_i.data_ptr(), None)
    assert misaligned == -1 and b"16-byte aligned" in lib.grace_topk_noalloc_strerror(misaligned)
