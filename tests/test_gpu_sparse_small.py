"""The single-CTA sparse exchange (``csrc/sparse_small.cu``: one tensor of at most 8192 elements) against plain
PyTorch restatements, over several steps of error feedback and several (emulated) ranks, and at the size where
the large kernel takes over."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _rand(n, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(n, generator=g) * 1e-3).to(_dev())


def _dense_topk(x, k):
    _, idx = torch.topk(x.abs(), k, sorted=False)
    out = torch.zeros_like(x)
    out[idx] = x[idx]
    return out


def _world(W, params):
    from grace_b200 import grace_from_params
    from grace_b200.communicator.fused import VirtualWorld

    def make(rank):
        p = dict(params)
        p.update(world_size=W, fused=True)
        return grace_from_params(p)

    return VirtualWorld(W, make, _dev())


@pytest.mark.parametrize("W", [1, 3])
@pytest.mark.parametrize("n", [1, 5, 127, 128, 1000, 4097, 8192, 8193])
def test_topk_residual_over_steps(W, n):
    ratio = 0.05
    k = max(1, int(n * ratio))
    vw = _world(W, {"compressor": "topk", "memory": "residual", "communicator": "allgather", "compress_ratio": ratio})
    residual = [torch.zeros(n, device=_dev()) for _ in range(W)]
    for step in range(4):                       # four steps: both send slots are reused
        grads = [_rand(n, seed=100 * step + r + n) for r in range(W)]
        outs = vw.step([g.clone() for g in grads], "w")
        vw.check()
        expect = torch.zeros(n, device=_dev())
        for r in range(W):
            acc = residual[r] + grads[r]
            sel = _dense_topk(acc, k)
            residual[r] = acc - sel
            expect += sel
        expect /= W
        for r in range(W):
            torch.testing.assert_close(outs[r], expect, rtol=1e-6, atol=1e-9)
            assert torch.equal(outs[r], outs[0])
            plan = next(iter(vw.comms[r]._plans.values()))
            assert torch.equal(plan.acc[:n], residual[r])


def test_ties_take_the_lowest_indices_and_exactly_k():
    n = 2000
    x = torch.full((n,), 0.25, device=_dev())
    x[1::2] = -0.25
    vw = _world(1, {"compressor": "topk", "memory": "none", "communicator": "allgather", "compress_ratio": 0.01})
    out = vw.step([x.clone()], "w")[0]
    assert out.nonzero().flatten().tolist() == list(range(20))
    assert torch.equal(out[:20], x[:20])
    z = vw.step([torch.zeros(n, device=_dev())], "w")[0]      # all zero: k entries of value 0 travel
    vw.check()
    assert not bool(z.any())


def test_dgc_momentum_correction_small():
    W, n, ratio, m = 2, 3000, 0.01, 0.9
    k = max(1, int(n * ratio))
    vw = _world(W, {"compressor": "dgc", "memory": "dgc", "communicator": "allgather", "compress_ratio": ratio,
                    "momentum": m})
    u = [torch.zeros(n, device=_dev()) for _ in range(W)]
    v = [torch.zeros(n, device=_dev()) for _ in range(W)]
    for step in range(3):
        grads = [_rand(n, seed=7 * step + r) for r in range(W)]
        outs = vw.step([g.clone() for g in grads], "w")
        vw.check()
        expect = torch.zeros(n, device=_dev())
        for r in range(W):
            u[r] = m * u[r] + grads[r]
            v[r] = v[r] + u[r]
            sel = _dense_topk(v[r], k)
            keep = sel == 0
            expect += sel
            u[r] = u[r] * keep
            v[r] = v[r] * keep
        torch.testing.assert_close(outs[0], expect / W, rtol=1e-6, atol=1e-9)
        plan = next(iter(vw.comms[0]._plans.values()))
        torch.testing.assert_close(plan.acc[:n], v[0], rtol=1e-6, atol=1e-9)
        torch.testing.assert_close(plan.u[:n], u[0], rtol=1e-6, atol=1e-9)


@pytest.mark.parametrize("strict", [False, True])
def test_threshold_small_and_overflow(strict):
    W, n, thr = 2, 6000, 2e-3
    params = {"compressor": "threshold", "memory": "residual", "communicator": "allgather", "threshold": thr}
    vw = _world(W, params)
    for c in vw.comms:
        c.compressor.strict = strict
    grads = [_rand(n, seed=r + 1) for r in range(W)]
    outs = vw.step([g.clone() for g in grads], "w")
    vw.check()
    expect = torch.zeros(n, device=_dev())
    for r in range(W):
        t = thr if strict else min(thr, grads[r].max().item())
        mask = grads[r].abs() > t if strict else grads[r].abs() >= t
        expect += torch.where(mask, grads[r], torch.zeros_like(grads[r]))
    torch.testing.assert_close(outs[0], expect / W, rtol=1e-6, atol=1e-9)
    # a slot holds a quarter of the elements: the first entries in index order travel, the rest stays in the residual
    vw = _world(1, params)
    x = torch.full((n,), 0.5, device=_dev())
    out = vw.step([x.clone()], "w")[0]
    vw.check()
    plan = next(iter(vw.comms[0]._plans.values()))
    sent = int((out != 0).sum())
    assert sent == plan.cap and bool((out[:sent] == 0.5).all())
    torch.testing.assert_close(out + plan.acc[:n], x)
    assert plan.channel.dropped() == n - sent


def test_bf16_gradient_small():
    n = 5000
    g = _rand(n, 3).to(torch.bfloat16)
    from grace_b200 import grace_from_params

    grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                             "compress_ratio": 0.02, "world_size": 1, "fused": True})
    out = grc.step(g.clone(), "w")
    grc.check()
    want = _dense_topk(g.float(), 100)
    torch.testing.assert_close(out.float(), want.to(torch.bfloat16).float(), rtol=0, atol=0)
