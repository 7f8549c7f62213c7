"""The reference's three extension modules keep their names and call signatures (``rdxtopk``, ``cnat_cuda``,
``qsgd_cuda``); on CPU tensors they run the torch implementations."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import cnat_cuda  # noqa: E402
import qsgd_cuda  # noqa: E402
import rdxtopk  # noqa: E402


def test_rdxtopk_topk_signature_and_result():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5000, generator=g)
    vals, idx = rdxtopk.topk(x.abs(), torch.arange(5000).int(), 50)
    assert vals.dtype == torch.float32 and idx.dtype == torch.int32 and vals.numel() == idx.numel() == 50
    assert torch.equal(vals.sort().values, torch.topk(x.abs(), 50).values.sort().values)
    assert torch.equal(x.abs()[idx.long()], vals)
    # indices are looked up through the tensor that was passed, as in the reference
    shifted = torch.arange(5000).int() + 7
    _, idx2 = rdxtopk.topk(x.abs(), shifted, 50)
    assert set(idx2.tolist()) == {i + 7 for i in idx.tolist()}
    # signed input: the k largest VALUES, not magnitudes
    v3, _ = rdxtopk.topk(x, torch.arange(5000).int(), 5)
    assert torch.equal(v3.sort().values, torch.topk(x, 5).values.sort().values)


def test_cnat_cuda_roundtrip_bounds():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4096, generator=g) * 1e-2
    code = cnat_cuda.compress(x)
    assert code.dtype == torch.uint8 and code.shape == x.shape
    y = cnat_cuda.decompress(code)
    ratio = y.abs() / x.abs()
    assert (y.sign() == x.sign()).all() and (ratio >= 0.5).all() and (ratio <= 2.0).all()   # neighbouring powers of two
    z = cnat_cuda.decompress(cnat_cuda.compress_deterministic(x))
    ratio = z.abs() / x.abs()
    assert (ratio > 0.66).all() and (ratio < 1.34).all()                                    # nearest of the two
    assert torch.equal(cnat_cuda.compress_deterministic(x), cnat_cuda.compress_deterministic(x))


def test_qsgd_cuda_signature_and_error_bound():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1000, generator=g)
    codes, norms = qsgd_cuda.compress(x, 64, 128)
    assert codes.dtype == torch.int8 and norms.dtype == torch.float64 and norms.numel() == 8
    assert codes.abs().max() <= 64
    y = qsgd_cuda.decompress(codes, norms, 64, 128)
    assert y.dtype == torch.float32 and y.shape == x.shape
    per_elem = norms.float().repeat_interleave(128)[:1000] / 64
    assert ((y - x).abs() <= per_elem + 1e-6).all()          # one quantisation step of the element's bucket
    zeros, zn = qsgd_cuda.compress(torch.zeros(256), 64, 128)
    assert not torch.isnan(qsgd_cuda.decompress(zeros, zn, 64, 128)).any()
