"""GPU tests of the fused kernels' options against plain PyTorch fp32 restatements: DGC gradient clipping computed
and exchanged inside the kernel, the strict threshold rule, bf16 / fp16 gradients read directly by the kernels,
one symmetric arena for many layouts, and the staged decode at eight (virtual) ranks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _rand(n, seed=0, scale=1e-3):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(n, generator=g) * scale).to(_dev())


def _world(W, params):
    from grace_b200 import grace_from_params
    from grace_b200.communicator.fused import VirtualWorld

    def make(rank):
        p = dict(params)
        p.update(world_size=W, fused=True)
        return grace_from_params(p)

    return VirtualWorld(W, make, _dev())


def _dense_topk(x, k):
    _, idx = torch.topk(x.abs(), k, sorted=False)
    out = torch.zeros_like(x)
    out[idx] = x[idx]
    return out


@pytest.mark.parametrize("W", [1, 2, 4])
def test_dgc_clipping_inside_the_kernel(W):
    """Clamp bound = sqrt(mean over ranks of sum g^2) per tensor, then momentum correction and exact top-k."""
    from grace_b200.ops.exchange import FlatLayout

    ratio, m = 0.02, 0.9
    names, numels = ["a", "b", "c"], [40_000, 513, 7_000]
    layout = FlatLayout(names, numels)
    vw = _world(W, {"compressor": "dgc", "memory": "dgc", "communicator": "allgather", "compress_ratio": ratio,
                    "momentum": m, "gradient_clipping": True})
    u = [[torch.zeros(n, device=_dev()) for n in numels] for _ in range(W)]
    v = [[torch.zeros(n, device=_dev()) for n in numels] for _ in range(W)]
    for step in range(3):
        flats = []
        grads = [[_rand(n, seed=1000 * step + 10 * r + i, scale=1.0) for i, n in enumerate(numels)] for r in range(W)]
        for i, n in enumerate(numels):   # one rank with a much larger norm: its outliers exceed the RMS-over-ranks bound
            grads[0][i][torch.arange(3, device=_dev()) * (n // 3)] *= 1000.0
        for r in range(W):
            f = torch.zeros(layout.total, device=_dev())
            for g, off, n in zip(grads[r], layout.offsets, numels):
                f[off:off + n] = g
            flats.append(f)
        outs = vw.step_flat(flats, layout, [torch.empty_like(f) for f in flats])
        vw.check()
        for i, (off, n) in enumerate(zip(layout.offsets, numels)):
            k = max(1, int(n * ratio))
            bound = torch.sqrt(sum((grads[r][i].double() ** 2).sum() for r in range(W)) / W).float()
            expect = torch.zeros(n, device=_dev())
            for r in range(W):
                g = torch.maximum(torch.minimum(grads[r][i], bound), -bound)
                u[r][i] = m * u[r][i] + g
                v[r][i] = v[r][i] + u[r][i]
                sel = _dense_topk(v[r][i], k)
                keep = sel == 0
                u[r][i] = u[r][i] * keep
                v[r][i] = v[r][i] * keep
                expect += sel
            expect /= W
            if W > 1:
                assert any(float(g[i].abs().max()) > float(bound) for g in grads), "the clamp must bind somewhere"
            for r in range(W):
                torch.testing.assert_close(outs[r][off:off + n], expect, rtol=1e-5, atol=2e-6 * float(expect.abs().max()))


def test_strict_threshold_rule_in_the_kernel():
    from grace_b200 import compressor as C, memory as M
    from grace_b200.communicator.fused import FusedExchange, VirtualWorld

    W, n, thr = 2, 60_000, 1.5
    vw = VirtualWorld(W, lambda r: FusedExchange(C.ThresholdCompressor(thr, strict=True), M.ResidualMemory(), W), _dev())
    assert vw.comms[0].supported(torch.zeros(4, device=_dev()))
    grads = [_rand(n, seed=r, scale=1.0) for r in range(W)]
    grads[0][7] = thr            # exactly on the threshold: kept by ">=", dropped by the strict rule
    grads[1][7] = 0.0
    outs = vw.step(grads, "w")
    vw.check()
    expect = sum(torch.where(g.abs() > thr, g, torch.zeros_like(g)) for g in grads) / W
    torch.testing.assert_close(outs[0], expect, rtol=0, atol=0)
    assert float(outs[0][7]) == 0.0
    # a tensor whose maximum is below the threshold sends nothing under the strict rule
    outs = vw.step([_rand(n, seed=9, scale=0.01) for _ in range(W)], "w2")
    vw.check()
    assert float(outs[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("codec", ["qsgd", "efsignsgd", "fp16", "topk"])
def test_sixteen_bit_gradients_are_read_by_the_kernels(dtype, codec):
    """Same result as casting the gradient to fp32 first (what the kernel does on load), output in the input's type."""
    from grace_b200 import grace_from_params

    params = {"qsgd": dict(compressor="qsgd", memory="residual", quantum_num=64),
              "efsignsgd": dict(compressor="efsignsgd", memory="efsignsgd", lr=0.1),
              "fp16": dict(compressor="fp16", memory="none"),
              "topk": dict(compressor="topk", memory="residual", compress_ratio=0.01)}[codec]
    n = 100_003 if codec != "topk" else 50_000
    a = grace_from_params(dict(params, communicator="allgather", world_size=1, fused=True, seed=5))
    b = grace_from_params(dict(params, communicator="allgather", world_size=1, fused=True, seed=5))
    for step in range(2):
        g16 = _rand(n, seed=step, scale=1.0).to(dtype).view(-1)
        out16 = a.step(g16.clone(), "w")
        out32 = b.step(g16.float(), "w")
        a.check(); b.check()
        assert out16.dtype == dtype and out16.shape == g16.shape
        if codec == "topk":
            # 16-bit data is full of equal magnitudes and ties at the k-th place are broken arbitrarily, so the two
            # runs may pick different places: check the selection against the accumulator it was made from
            k = max(1, int(n * 0.01))
            acc = g16.float() + (0 if step == 0 else prev_res)
            nz = out16 != 0
            assert int(nz.sum()) == k
            assert torch.equal(out16[nz].float(), acc[nz].to(dtype).float())
            assert float(acc[nz].abs().min()) >= float(acc[~nz].abs().max())      # a true top-k of the accumulator
            prev_res = next(iter(a._plans.values())).acc[:n].clone()
            assert torch.equal(prev_res, torch.where(nz, torch.zeros_like(acc), acc))
        else:
            torch.testing.assert_close(out16, out32.to(dtype), rtol=0, atol=0)
    pa = next(iter(a._plans.values())); pb = next(iter(b._plans.values()))
    if pa.acc is not None and codec != "topk":
        torch.testing.assert_close(pa.acc, pb.acc, rtol=0, atol=0)       # residuals stay fp32 and identical


def test_many_layouts_share_one_arena():
    vw = _world(2, {"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": 0.1})
    for i in range(100):
        n = 300 + 8 * i
        outs = vw.step([_rand(n, seed=i), _rand(n, seed=1000 + i)], "t%d" % i)
    vw.check()
    assert len(vw._arena.segments) == 1                # 100 plans, one allocation per (virtual) rank
    assert len(vw.comms[0]._plans) == 100
    assert torch.isfinite(outs[0]).all()


@pytest.mark.parametrize("codec,extra", [("qsgd", {"quantum_num": 64}), ("natural", {"deterministic": True}),
                                         ("u8bit", {}), ("terngrad", {}), ("signsgd", {}), ("efsignsgd", {"lr": 0.1}),
                                         ("onebit", {})])
def test_staged_decode_matches_single_rank_decodes(codec, extra):
    """Eight ranks through the staged decode: the aggregate equals the combination of every rank's own decode
    (each obtained from a one-rank exchange of the same gradient with the same seed)."""
    from grace_b200 import grace_from_params

    W, n = 8, 70_001
    mem = "efsignsgd" if codec == "efsignsgd" else "none"
    base = dict(compressor=codec, memory=mem, communicator="allgather", seed=3, **extra)
    vw = _world(W, base)
    grads = [_rand(n, seed=50 + r, scale=1.0) for r in range(W)]
    outs = vw.step([g.clone() for g in grads], "w")
    vw.check()
    singles = []
    for r in range(W):
        one = grace_from_params(dict(base, world_size=1, fused=True))
        singles.append(one.step(grads[r].clone(), "w"))
        one.check()
    if codec == "signsgd":
        votes = sum(singles)
        expect = torch.where(votes >= 0, torch.ones_like(votes), -torch.ones_like(votes))
        assert torch.equal(outs[0], expect)
    elif codec == "efsignsgd":
        torch.testing.assert_close(outs[0], sum(singles), rtol=1e-5, atol=2e-5)   # sums of +-mean/lr ~ 8 that cancel
    else:
        torch.testing.assert_close(outs[0], sum(singles) / W, rtol=1e-5, atol=1e-7)
    for r in range(1, W):
        assert torch.equal(outs[0], outs[r])


@pytest.mark.parametrize("bucket,q", [(32, 64), (64, 127), (256, 64), (512, 300), (100, 1000), (128, 255)])
@pytest.mark.parametrize("W", [1, 2])
def test_general_qsgd_buckets_and_levels(bucket, q, W):
    """QSGD with any bucket size that is a multiple of 4 and more than 127 levels stays on the fused path: per bucket
    of each tensor, codes are integers in [-q, q], the decoded value is norm / q * code, its error is below one level,
    and the residual holds exactly what was not transmitted."""
    from grace_b200.ops.exchange import FlatLayout

    names, numels = ["a", "b"], [5000, 777]
    layout = FlatLayout(names, numels)
    vw = _world(W, {"compressor": "qsgd", "memory": "residual", "communicator": "allgather", "quantum_num": q,
                    "bucket_size": bucket, "seed": 11})
    assert vw.comms[0]._kind == "quant"
    flats, grads = [], []
    for r in range(W):
        gs = [_rand(n, seed=31 * r + i, scale=1.0) for i, n in enumerate(numels)]
        f = torch.zeros(layout.total, device=_dev())
        for g, off, n in zip(gs, layout.offsets, numels):
            f[off:off + n] = g
        flats.append(f)
        grads.append(gs)
    outs = vw.step_flat([f.clone() for f in flats], layout, [torch.empty_like(f) for f in flats])
    vw.check()
    for i, (off, n) in enumerate(zip(layout.offsets, numels)):
        expect = torch.zeros(n, device=_dev())
        for r in range(W):
            g = grads[r][i]
            res = next(iter(vw.comms[r]._plans.values())).acc[off:off + n]
            dec = g - res                                   # what rank r transmitted (error-feedback identity)
            pad = (-n) % bucket
            gb = torch.nn.functional.pad(g, (0, pad)).view(-1, bucket)
            db = torch.nn.functional.pad(dec, (0, pad)).view(-1, bucket)
            norms = gb.norm(dim=1, keepdim=True)
            codes = db * q / norms.clamp_min(1e-30)
            assert float((codes - codes.round()).abs().max()) < 2e-3           # integer levels
            assert float(codes.abs().max()) <= q + 1e-3
            assert float(((db - gb).abs() * q / norms.clamp_min(1e-30)).max()) < 1.0 + 1e-3   # within one level
            expect += dec
        torch.testing.assert_close(outs[0][off:off + n], expect / W, rtol=1e-5, atol=1e-6)
        for r in range(1, W):     # (the gaps between tensors are nobody's business)
            assert torch.equal(outs[0][off:off + n], outs[r][off:off + n])
