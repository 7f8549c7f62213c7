"""GPU tests of the fused quantised exchange against PyTorch/NumPy fp32
restatements that consume the same Philox stream."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _rand(n, seed=0, scale=1e-3):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(n, generator=g) * scale).to(_dev())


def _uniform(n, seed, step):
    from grace_b200.utils.philox import uniform

    return torch.from_numpy(uniform(n, seed, step)).to(_dev())


def _world(W, params):
    from grace_b200 import grace_from_params
    from grace_b200.communicator.fused import VirtualWorld

    def make(rank):
        p = dict(params)
        p.update(world_size=W, fused=True)
        return grace_from_params(p)

    return VirtualWorld(W, make, _dev())


def _plan(vw, r=0):
    return next(iter(vw.comms[r]._plans.values()))


@pytest.mark.parametrize("n", [1, 100, 128, 129, 5000, 200_001])
def test_qsgd_compress_matches_oracle(n):
    from grace_b200.ops.quant import qsgd_compress

    q = 64
    x = _rand(n, n)
    seed, step = 1234567, 3
    codes, norms = qsgd_compress(x, q, 128, "t", seed=seed, step=step)
    pad = (-n) % 128
    xb = torch.cat([x, x.new_zeros(pad)]).view(-1, 128)
    ref_norm = xb.pow(2).sum(1).sqrt()
    torch.testing.assert_close(norms, ref_norm, rtol=1e-5, atol=0)
    norm_e = norms.repeat_interleave(128)[:n]
    u = _uniform(n, seed, step)
    lf = q / torch.where(norm_e > 0, norm_e, torch.ones_like(norm_e)) * x.abs()
    level = lf.floor() + (u < (lf - lf.floor())).float()
    ref = (level * x.sign()).to(torch.int8)
    assert torch.equal(codes, ref)
    assert codes.abs().max() <= q


def test_qsgd_unbiased():
    from grace_b200.ops.quant import qsgd_compress

    n, q = 4096, 16
    x = _rand(n, 1)
    acc = torch.zeros(n, device=_dev())
    trials = 400
    for t in range(trials):
        codes, norms = qsgd_compress(x, q, 128, "t", seed=99, step=t)
        acc += norms.repeat_interleave(128)[:n] / q * codes.float()
    mean = acc / trials
    sigma = (norms.repeat_interleave(128)[:n] / q) * 0.5 / np.sqrt(trials)
    assert torch.all((mean - x).abs() <= 5 * sigma + 1e-12)


@pytest.mark.parametrize("W", [1, 2, 4])
def test_qsgd_exchange_with_residual(W):
    n, q = 33_333, 64
    vw = _world(W, {"compressor": "qsgd", "memory": "residual", "communicator": "allgather", "quantum_num": q})
    residual = [torch.zeros(n, device=_dev()) for _ in range(W)]
    for step in range(2):
        grads = [_rand(n, 50 * step + r) for r in range(W)]
        outs = vw.step(grads, "w")
        vw.check()
        expect = torch.zeros(n, device=_dev())
        for r in range(W):
            acc = residual[r] + grads[r]
            pad = (-n) % 128
            norms = torch.cat([acc, acc.new_zeros(pad)]).view(-1, 128).pow(2).sum(1).sqrt()
            norm_e = norms.repeat_interleave(128)[:n]
            u = _uniform(n, _plan(vw, r).seed, step)
            lf = q / norm_e * acc.abs()
            level = lf.floor() + (u < (lf - lf.floor())).float()
            dec = norm_e / q * (level * acc.sign())
            residual[r] = acc - dec
            expect += dec
        expect /= W
        for r in range(W):
            # norms are reduced in a different order than torch: allow one level flip per ~1e5 elements
            diff = (outs[r] - expect).abs()
            assert (diff > 1e-7).float().mean() < 1e-3
            assert torch.equal(outs[0], outs[r])


def _natural_oracle(x, u):
    from grace_b200.compressor.natural import natural_decode, natural_encode

    code = natural_encode(x.cpu(), u.cpu())
    return code.to(x.device), natural_decode(code).to(x.device)


@pytest.mark.parametrize("n", [5, 128, 10_001])
def test_natural_compress_matches_oracle(n):
    from grace_b200.ops.quant import natural_compress

    x = _rand(n, n, scale=1.0)
    x[0] = 0.0
    code = natural_compress(x, "t", seed=42, step=0)
    ref_code, ref_dec = _natural_oracle(x, _uniform(n, 42, 0))
    assert torch.equal(code, ref_code)
    # decode of every non-zero code is within a factor of two below/above
    nz = x != 0
    ratio = (ref_dec[nz] / x[nz])
    assert torch.all((ratio > 0.5 - 1e-6) & (ratio <= 2.0 + 1e-6))
    det = natural_compress(x, "t", deterministic=True, seed=0, step=0)
    ref_det, _ = _natural_oracle(x, torch.where(((x.view(torch.int32) & 0x7FFFFF) > 0x400000), 0.0, 1.0).to(x.device))
    assert torch.equal(det, ref_det)


def test_terngrad_compress_properties():
    from grace_b200.ops.quant import terngrad_compress

    n = 50_000
    x = _rand(n, 3)
    tern, scale = terngrad_compress(x, "t", seed=5, step=1)
    assert set(tern.unique().tolist()) <= {-1, 0, 1}
    std = (x - x.mean()).pow(2).mean().sqrt()
    c = 2.5 * std
    s_ref = x.clamp(-c, c).abs().max()
    torch.testing.assert_close(scale[0], s_ref, rtol=1e-5, atol=0)
    u = _uniform(n, 5, 1)
    mag = x.abs().clamp(max=c.item())
    ref = torch.where(u * scale[0] < mag, x.sign(), torch.zeros_like(x)).to(torch.int8)
    assert (tern != ref).float().mean() < 1e-4  # scale differs in the last ulp at most


CODECS = [
    ("terngrad", "none", {}),
    ("natural", "residual", {}),
    ("u8bit", "residual", {}),
    ("signsgd", "none", {}),
    ("signum", "none", {"momentum": 0.9}),
    ("efsignsgd", "efsignsgd", {"lr": 0.1}),
    ("onebit", "residual", {}),
    ("fp16", "none", {}),
    ("none", "none", {}),
]


@pytest.mark.parametrize("name,memory,extra", CODECS)
@pytest.mark.parametrize("W", [1, 3])
def test_codec_exchange_matches_python_compressor(name, memory, extra, W):
    """Fused result == aggregate of the Python compressor's decompress over ranks,
    with the Python compressor fed the kernel's Philox stream."""
    from grace_b200 import grace_from_params

    n = 20_011
    params = {"compressor": name, "memory": memory, "communicator": "allgather", **extra}
    vw = _world(W, params)
    # python-side replicas (CPU semantics on GPU tensors through torch ops)
    refs = [grace_from_params({**params, "world_size": W}) for _ in range(W)]
    for step in range(2):
        grads = [_rand(n, 31 * step + r, scale=1e-2) for r in range(W)]
        outs = vw.step([g.clone() for g in grads], "w")
        vw.check()
        dec = []
        for r in range(W):
            comp, mem = refs[r].compressor, refs[r].memory
            seed = _plan(vw, r).seed
            comp.uniform_fn = lambda like, nm, s=seed, st=step: _uniform(like.numel(), s, st).cpu()
            t = mem.compensate(grads[r].cpu(), "w")
            payload, ctx = comp.compress(t, "w")
            mem.update(t, "w", comp, payload, ctx)
            dec.append(comp.decompress(payload, ctx).float().to(_dev()))
        agg = refs[0].compressor.aggregate(dec)
        expect = agg / W if refs[0].compressor.average else agg
        tol = dict(rtol=2e-5, atol=1e-7)
        if name in ("terngrad", "onebit", "efsignsgd", "u8bit"):
            # per-tensor scalars are reduced in a different order than torch
            frac = ((outs[0] - expect).abs() > 1e-5 * expect.abs().max()).float().mean()
            assert frac < 2e-3, frac
        else:
            torch.testing.assert_close(outs[0], expect, **tol)
        for r in range(1, W):
            assert torch.equal(outs[0], outs[r])
        if hasattr(refs[0].memory, "residuals") and name in ("natural",):
            torch.testing.assert_close(_plan(vw, 0).acc[:n], refs[0].memory.residuals["w"].to(_dev()), rtol=1e-5, atol=1e-8)


def _a2a_world(W, params):
    from grace_b200 import grace_from_params
    from grace_b200.communicator.fused import VirtualWorld

    def make(rank):
        p = dict(params)
        p.update(world_size=W, fused=True, communicator="alltoall")
        return grace_from_params(p)

    return VirtualWorld(W, make, _dev())


@pytest.mark.parametrize("W", [2, 3, 4])
def test_two_phase_mode_dense_and_natural(W):
    """Compressed reduce-scatter + all-gather: exact for the dense codec, and equal to
    decode -> sum -> re-encode -> decode for deterministic natural compression."""
    from grace_b200.compressor.natural import natural_decode, natural_encode

    n = 50_001
    grads = [_rand(n, 11 * r + 1, scale=1e-2) for r in range(W)]
    vw = _a2a_world(W, {"compressor": "none", "memory": "none"})
    assert vw.comms[0].mode == "alltoall"
    outs = vw.step([g.clone() for g in grads], "w")
    vw.check()
    assert next(iter(vw.comms[0]._plans.values())).alltoall
    torch.testing.assert_close(outs[0], sum(grads) / W, rtol=1e-6, atol=1e-9)
    for r in range(1, W):
        assert torch.equal(outs[0], outs[r])

    from grace_b200 import grace_from_params
    from grace_b200.communicator.fused import VirtualWorld

    def make(rank):
        c = grace_from_params({"compressor": "natural", "memory": "none", "communicator": "alltoall",
                               "world_size": W, "fused": True})
        c.compressor.deterministic = True
        return c

    vw = VirtualWorld(W, make, _dev())
    outs = vw.step([g.clone() for g in grads], "w")
    vw.check()

    def det_code(x):
        prob = ((x.view(torch.int32) & 0x7FFFFF) > 0x400000)
        return natural_encode(x, torch.where(prob, 0.0, 1.0).to(x.device))

    total = sum(natural_decode(det_code(g.cpu())) for g in grads)
    expect = natural_decode(det_code(total.contiguous())) / W
    torch.testing.assert_close(outs[0].cpu(), expect, rtol=0, atol=0)


def test_two_phase_mode_qsgd_close_to_mean():
    W, n = 4, 100_000
    grads = [_rand(n, 5 * r + 2, scale=1e-2) for r in range(W)]
    vw = _a2a_world(W, {"compressor": "qsgd", "memory": "residual", "quantum_num": 127})
    outs = vw.step([g.clone() for g in grads], "w")
    vw.check()
    mean = sum(grads) / W
    assert ((outs[0] - mean).norm() / mean.norm()).item() < 0.12
    for r in range(1, W):
        assert torch.equal(outs[0], outs[r])


def test_fused_state_dict_resume_is_bit_identical():
    """Save the fused communicator's state, rebuild it, load: the next exchange (same Philox
    counters, same residuals) must give bit-identical results."""
    from grace_b200 import grace_from_params

    n = 40_000
    params = {"compressor": "qsgd", "memory": "residual", "communicator": "allgather", "quantum_num": 64,
              "world_size": 1, "fused": True, "seed": 11}
    a = grace_from_params(params)
    xs = [_rand(n, 70 + i, scale=1e-2) for i in range(4)]
    a.step(xs[0].clone(), "w"); a.step(xs[1].clone(), "w")
    a.check()
    state = a.state_dict()
    assert "residuals" in state["memory"] and "w" in state["memory"]["residuals"]
    b = grace_from_params(params)
    b.load_state_dict(state)
    out_a = a.step(xs[2].clone(), "w")
    out_b = b.step(xs[2].clone(), "w")
    a.check(); b.check()
    assert torch.equal(out_a, out_b)
    pa, pb = next(iter(a._plans.values())), next(iter(b._plans.values()))
    assert torch.equal(pa.acc, pb.acc)


def test_guard_bands_stay_intact(monkeypatch):
    """GRACE_GUARD=1 surrounds the send slots with poison bytes; every codec must leave them alone."""
    monkeypatch.setenv("GRACE_GUARD", "1")
    n = 12_345
    for name, memory in (("qsgd", "residual"), ("terngrad", "none"), ("signsgd", "none"), ("topk", "residual"),
                         ("fp16", "none")):
        vw = _world(2, {"compressor": name, "memory": memory, "communicator": "allgather", "compress_ratio": 0.05,
                        "quantum_num": 64})
        vw.step([_rand(n, r) for r in range(2)], "w")
        plan = _plan(vw)
        assert plan.channel.guard and len(plan.channel.guard_off) == 3
        vw.check()   # raises if a guard band changed


@pytest.mark.parametrize("comp,extra", [("qsgd", {"quantum_num": 64}), ("natural_cuda", {})])
def test_pipelined_exchange_gives_the_bits_of_the_phase_by_phase_kernel(comp, extra):
    """One rank, pipelined mode forced (tiles drawn from the queue, chunk counters, chunk flags to itself) against
    the phase-by-phase kernel over a flat buffer of several tensors whose sizes are no multiples of a tile: outputs
    and residuals must agree bit for bit, step after step."""
    from grace_b200 import grace_from_params
    from grace_b200.ops.exchange import FlatLayout

    dev = torch.device("cuda")
    layout = FlatLayout.from_named([("a", 250_000), ("b", 64), ("c", 2_234_567), ("d", 9)])
    pair = [grace_from_params({"compressor": comp, "memory": "residual", "communicator": "allgather", "world_size": 1,
                               "fused": True, "timeout_ms": 3000, "pipeline": mode, **extra}) for mode in ("force", False)]
    for step in range(4):
        g = torch.Generator().manual_seed(step)
        flat = torch.zeros(layout.total, device=dev)
        for o, c in zip(layout.offsets, layout.numels):
            flat[o:o + c] = (torch.randn(c, generator=g) * 1e-3).to(dev)
        a, b = flat.clone(), flat.clone()
        pair[0].step_flat(a, layout)
        pair[1].step_flat(b, layout)
        pair[0].check()
        pair[1].check()
        assert torch.equal(a, b), step
    plans = [next(iter(c._plans.values())) for c in pair]
    assert plans[0].pipeline is not None and plans[1].pipeline is None
    assert torch.equal(plans[0].acc, plans[1].acc)
    # one tile in one chunk, and two chunks of one tile: the ends of the queue arithmetic
    for small in ([("s", 5000)], [("s", 12_000), ("t", 3)]):
        small_layout = FlatLayout.from_named(small)
        pair = [grace_from_params({"compressor": comp, "memory": "residual", "communicator": "allgather",
                                   "world_size": 1, "fused": True, "timeout_ms": 3000, "pipeline": mode, **extra})
                for mode in ("force", False)]
        for step in range(2):
            flat = torch.zeros(small_layout.total, device=dev)
            for o, c in zip(small_layout.offsets, small_layout.numels):
                flat[o:o + c] = torch.randn(c, device=dev) * 1e-3
            a, b = flat.clone(), flat.clone()
            pair[0].step_flat(a, small_layout)
            pair[1].step_flat(b, small_layout)
            pair[0].check()
            assert torch.equal(a, b), (small, step)
    # a bf16 gradient buffer goes through the same typed loads and stores
    pair = [grace_from_params({"compressor": comp, "memory": "residual", "communicator": "allgather", "world_size": 1,
                               "fused": True, "timeout_ms": 3000, "pipeline": mode, **extra}) for mode in ("force", False)]
    flat = (torch.randn(layout.total, device=dev) * 1e-3).to(torch.bfloat16)
    a, b = flat.clone(), flat.clone()
    pair[0].step_flat(a, layout)
    pair[1].step_flat(b, layout)
    pair[0].check()
    assert torch.equal(a, b)
