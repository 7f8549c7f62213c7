"""CPU tests of the compressor / memory semantics (the reference ships none;
these pin the numeric contracts of its algorithms)."""
import math

import numpy as np
import pytest
import torch

from grace_b200 import compressor as C
from grace_b200 import memory as M


def _x(n=1000, seed=0, scale=1e-2):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * scale


def test_none_and_fp16_roundtrip():
    x = _x().view(10, 100)
    p, ctx = C.NoneCompressor().compress(x, "a")
    assert torch.equal(C.NoneCompressor().decompress(p, ctx), x)
    c = C.FP16Compressor()
    p, ctx = c.compress(x, "a")
    assert p[0].dtype == torch.float16
    out = c.decompress(p, ctx)
    assert out.dtype == torch.float32 and torch.allclose(out, x, rtol=1e-3, atol=1e-6)


@pytest.mark.parametrize("ratio", [0.001, 0.01, 0.3, 1.0])
def test_topk_exact_k_and_values(ratio):
    x = _x(5000).view(50, 100)
    c = C.TopKCompressor(ratio)
    (vals, idx), ctx = c.compress(x, "a")
    k = max(1, int(5000 * ratio))
    assert vals.numel() == k and idx.dtype == torch.int32
    dense = c.decompress((vals, idx), ctx)
    assert dense.shape == x.shape
    kth = x.abs().flatten().topk(k).values[-1]
    assert torch.all(dense[dense != 0].abs() >= kth)
    assert (dense != 0).sum() == k


def test_randomk_same_indices_for_same_name_and_step():
    a, b = C.RandomKCompressor(0.1), C.RandomKCompressor(0.1)
    x, y = _x(seed=1), _x(seed=2)
    (_,), (ia, _, _) = a.compress(x, "layer.weight")
    (_,), (ib, _, _) = b.compress(y, "layer.weight")
    assert torch.equal(ia, ib)
    (_,), (ia2, _, _) = a.compress(x, "layer.weight")
    assert not torch.equal(ia, ia2)  # the step is part of the seed
    assert a.state_dict()["global_step"] == 2
    (v,), ctx = b.compress(y, "other")
    dense = b.decompress([v], ctx)
    assert dense.shape == y.shape


def test_threshold_selects_by_magnitude_and_handles_small_max():
    x = torch.tensor([0.5, -0.02, 0.005, -0.3, 0.0])
    c = C.ThresholdCompressor(0.01)
    (vals, idx), ctx = c.compress(x, "a")
    assert idx.tolist() == [0, 1, 3]
    assert torch.equal(c.decompress((vals, idx), ctx), torch.tensor([0.5, -0.02, 0.0, -0.3, 0.0]))
    small = torch.tensor([0.001, -0.004, 0.002])
    (vals, idx), _ = c.compress(small, "b")  # threshold falls back to max(x) = 0.002
    assert idx.tolist() == [1, 2]


@pytest.mark.parametrize("mode", ["sampled", "exact"])
def test_dgc_count_in_band_and_memory_masks(mode):
    torch.manual_seed(0)
    n, ratio = 100_000, 0.01
    c = C.DgcCompressor(ratio, mode=mode)
    mem = M.DgcMemory(0.9, False, 1)
    g1, g2 = _x(n, 1), _x(n, 2)
    t = mem.compensate(g1, "w")
    (vals, idx), ctx = c.compress(t, "w")
    assert 0.7 * ratio * n <= vals.numel() <= 1.3 * ratio * n
    mem.update(t, "w", c, (vals, idx), ctx)
    assert torch.all(mem.gradients["w"][idx.long()] == 0) and torch.all(mem.residuals["w"][idx.long()] == 0)
    u1, v1 = mem.residuals["w"].clone(), mem.gradients["w"].clone()
    t2 = mem.compensate(g2, "w")
    torch.testing.assert_close(mem.residuals["w"], 0.9 * u1 + g2)
    torch.testing.assert_close(t2, v1 + 0.9 * u1 + g2)


def test_dgc_clipping_runs_single_process():
    mem = M.DgcMemory(0.9, True, 1)
    g = torch.tensor([3.0, -4.0, 0.1])
    out = mem.compensate(g, "w")
    assert out.abs().max() <= 5.0 + 1e-6


def test_qsgd_levels_bounds_unbiased_and_zero_bucket():
    q = 16
    c = C.QSGDCompressor(q, 128)
    x = _x(1000)
    x[256:384] = 0  # a zero-norm bucket must not produce NaN
    (code, norms), ctx = c.compress(x, "a")
    assert code.dtype == torch.int8 and code.abs().max() <= q and norms.numel() == math.ceil(1000 / 128)
    dec = c.decompress((code, norms), ctx)
    assert torch.isfinite(dec).all() and torch.all(dec[256:384] == 0)
    acc = torch.zeros_like(x)
    for _ in range(300):
        p, ctx = c.compress(x, "a")
        acc += c.decompress(p, ctx)
    step = norms.repeat_interleave(128)[:1000] / q
    assert torch.all(((acc / 300) - x).abs() <= 5 * step * 0.5 / math.sqrt(300) + 1e-9)
    big = C.QSGDCompressor(200)
    (code, _), _ = big.compress(x, "a")
    assert code.dtype == torch.float16


def test_terngrad_values_and_scale():
    c = C.TernGradCompressor()
    x = _x(5000)
    (t, s), ctx = c.compress(x, "a")
    assert set(t.unique().tolist()) <= {-1, 0, 1} and t.dtype == torch.int8
    std = (x - x.mean()).pow(2).mean().sqrt()
    assert torch.isclose(s[0], x.clamp(-2.5 * std, 2.5 * std).abs().max())
    assert torch.equal(c.decompress((t, s), ctx), t.float() * s)


def test_sign_family():
    x = torch.tensor([0.5, -0.2, 0.0, -3.0])
    s = C.SignSGDCompressor()
    (bits,), ctx = s.compress(x, "a")
    assert bits.tolist() == [1, 0, 1, 0] and not s.average
    d = s.decompress([bits], ctx)
    assert d.tolist() == [1, -1, 1, -1]
    votes = s.aggregate([torch.tensor([1.0, -1, 1, -1]), torch.tensor([-1.0, -1, 1, 1])])
    assert votes.tolist() == [1, -1, 1, 1]  # ties go to +1
    m = C.SignumCompressor(0.9)
    m.compress(x, "a")
    assert torch.equal(m.momentums["a"], x)
    m.compress(-x, "a")
    torch.testing.assert_close(m.momentums["a"], 0.1 * (-x) + 0.9 * x)
    e = C.EFSignSGDCompressor(0.1)
    (mean, bits), ctx = e.compress(x, "a")
    assert torch.isclose(mean, x.abs().mean())
    agg = e.aggregate([e.decompress((mean, bits), ctx)] * 2)
    torch.testing.assert_close(agg, 2 * mean * torch.tensor([1.0, -1, 1, -1]) / 0.1)


def test_onebit_corrected_decode():
    x = torch.tensor([1.0, 3.0, -2.0, -4.0, 0.0])
    c = C.OneBitCompressor()
    p, ctx = c.compress(x, "a")
    d = c.decompress(p, ctx)
    torch.testing.assert_close(d, torch.tensor([4 / 3, 4 / 3, -3.0, -3.0, 4 / 3]))
    p, ctx = c.compress(torch.tensor([1.0, 2.0]), "b")  # empty negative set
    assert torch.isfinite(c.decompress(p, ctx)).all()


def test_natural_code_table_and_unbiased():
    from grace_b200.compressor.natural import natural_decode, natural_encode

    x = torch.tensor([0.0, 1.0, -1.0, 0.75, 2.0 ** -120, 2.0 ** 30, -3.0])
    lo = natural_encode(x, torch.ones_like(x))     # never round up
    hi = natural_encode(x, torch.zeros_like(x))    # round up whenever the mantissa is non-zero
    assert lo[0] == 0 and hi[0] == 0
    assert natural_decode(lo).tolist()[:4] == [0.0, 1.0, -1.0, 0.5]
    assert natural_decode(hi).tolist()[:4] == [0.0, 1.0, -1.0, 1.0]
    assert natural_decode(lo)[4] == 0 and natural_decode(lo)[5] == 2.0 ** 17  # flush / saturate
    assert natural_decode(lo)[6] == -2.0 and natural_decode(hi)[6] == -4.0
    c = C.NaturalCompressor()
    x = _x(2000, scale=1.0)
    acc = torch.zeros_like(x)
    for _ in range(400):
        p, ctx = c.compress(x, "a")
        acc += c.decompress(p, ctx)
    assert ((acc / 400 - x).abs() <= 5 * x.abs() / math.sqrt(400) + 1e-9).all()
    det = C.NaturalCompressor(deterministic=True)
    (code,), ctx = det.compress(torch.tensor([0.74, 0.76, 1.6]), "d")
    assert det.decompress([code], ctx).tolist() == [0.5, 1.0, 2.0]


def test_u8bit_table_and_roundtrip():
    from grace_b200.compressor.u8bit import DICT128

    assert DICT128.numel() == 128 and torch.all(DICT128[1:] > DICT128[:-1])
    for i, v in ((0, 1.5000001e-06), (7, 1.4375e-04), (31, 1.109375e-02), (63, 1.0546875e-01), (127, 9.9570298e-01)):
        assert abs(DICT128[i].item() - v) <= 1e-7 * max(1, v / 1e-6) * 1e-1 + 2e-8
    c = C.U8bitCompressor()
    x = _x(4000)
    (code, s), ctx = c.compress(x, "a")
    assert code.dtype == torch.int8 and code.abs().max() <= 126
    d = c.decompress((code, s), ctx)
    assert torch.all(d.abs() <= x.abs() + 1e-12)          # lower bin edge
    nz = code != 0
    assert torch.all(d[nz].sign() == x[nz].sign())
    rel = (x[nz].abs() - d[nz].abs()) / x[nz].abs()
    assert rel.max() < 0.65


def test_powersgd_rank_and_warm_start():
    torch.manual_seed(0)
    a, b = torch.randn(64, 4), torch.randn(4, 48)
    m = a @ b  # exactly rank 4
    c = C.PowerSGDCompressor(rank=4, use_memory=True, world_size=1)
    vec = torch.randn(10)
    p, ctx = c.compress(vec, "bias")
    assert ctx is None and c.decompress(p, ctx) is vec
    err = []
    for _ in range(3):
        p, ctx = c.compress(m, "w")
        assert p == [] and ctx[0].shape == (64, 4) and ctx[1].shape == (48, 4)
        err.append(((c.decompress(p, ctx) - m).norm() / m.norm()).item())
    assert err[-1] < 1e-4
    mem = M.PowerSGDMemory(c.q_memory, 4)
    t = mem.compensate(m, "w2")
    p, ctx = c.compress(t, "w2")
    mem.update(t, "w2", c, p, ctx)
    torch.testing.assert_close(mem.residuals["w2"], t - c.decompress(p, ctx))


def test_second_tier_codecs_roundtrip():
    x = _x(3000)
    a = C.AdaqCompressor(0.05)
    p, ctx = a.compress(x, "a")
    d = a.decompress(p, ctx)
    assert p[0].dtype == torch.int32 and set(d.unique().numel() for _ in [0]) == {3}
    s = C.SketchCompressor(64)
    p, ctx = s.compress(x, "a")
    d = s.decompress(p, ctx)
    assert p[0].dtype == torch.uint8 and (d - x).abs().mean() < x.abs().mean() * 0.2
    i = C.INCEPTIONNCompressor(2e-10)
    y = torch.cat([x, torch.tensor([1.5, -3.0, 1e-12])])
    p, ctx = i.compress(y, "a")
    d = i.decompress(p, ctx)
    assert d[-3] == 1.5 and d[-2] == -3.0 and d[-1] == 0
    assert (d[:3000] - x).abs().max() <= 2.0 ** -7
    from grace_b200.compressor.packing import decode_byte, encode_byte

    cls = torch.tensor([0, 1, 2, 3, 3, 2])
    assert torch.equal(decode_byte(encode_byte(cls), 6), cls)


def test_residual_memory_first_step_and_identity():
    mem = M.ResidualMemory(beta=0.5, gamma=2.0)
    c = C.TopKCompressor(0.1)
    g = _x(100)
    t = mem.compensate(g, "w")
    assert t is g  # gamma is not applied before a residual exists
    p, ctx = c.compress(t, "w")
    mem.update(t, "w", c, p, ctx)
    torch.testing.assert_close(mem.residuals["w"] + c.decompress(p, ctx), g)
    g2 = _x(100, 5)
    torch.testing.assert_close(mem.compensate(g2, "w"), 0.5 * mem.residuals["w"] + 2.0 * g2)
    ef = M.EFSignSGDMemory(0.1)
    assert ef.compensate(g, "w") is g


def test_philox_matches_known_answers():
    from grace_b200.utils.philox import philox4x32, uniform

    assert [int(v) for v in philox4x32(0, 0, 0, 0, 0, 0)] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    u = uniform(10_000, 7, 3)
    assert u.dtype == np.float32 and 0 <= u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.02
