"""The two engines of the exchange protocol against each other: the sm_100a kernels on the GPU and the host
engine (``csrc/host_exchange.cpp``) on the CPU get the same gradients, names and seed.  Integer decisions (which
entries travel, which sign wins) must agree exactly; stochastic rounding draws the same Philox words on both
sides, so QSGD agrees except where a bucket norm differs in its last bit (the warp adds the squares in a tree,
the host one after the other)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(params, n, steps=2, seed=0):
    from grace_b200 import grace_from_params
    from grace_b200.communicator.host import ThreadWorld

    gs = [torch.randn(n, generator=torch.Generator().manual_seed(50 * seed + s)) * 1e-3 for s in range(steps)]
    dev = grace_from_params(dict(params, world_size=1, fused=True))
    out_dev = [dev.step(g.cuda(), "layer.weight").cpu() for g in gs]
    dev.check()

    def body(view):
        host = grace_from_params(dict(params, world_size=1, host_protocol=True, host_world=view))
        return [host.step(g.clone(), "layer.weight") for g in gs]

    return out_dev, ThreadWorld(1).run(body)[0]


@pytest.mark.parametrize("n", [1000, 128 * 1024 + 5])
def test_topk_residual_same_entries(n):
    dev, host = _pair({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                       "compress_ratio": 0.01}, n, steps=3)
    for a, b in zip(dev, host):
        assert torch.equal(a, b)


def test_sign_vote_and_dense_are_identical():
    dev, host = _pair({"compressor": "signsgd", "memory": "none", "communicator": "allgather"}, 70_001)
    assert all(torch.equal(a, b) for a, b in zip(dev, host))
    dev, host = _pair({"compressor": "none", "memory": "none", "communicator": "allgather"}, 70_001)
    assert all(torch.equal(a, b) for a, b in zip(dev, host))


def test_efsign_agrees_to_rounding():
    dev, host = _pair({"compressor": "efsignsgd", "memory": "efsignsgd", "communicator": "allgather", "lr": 0.1},
                      100_000, steps=3)
    for a, b in zip(dev, host):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-9)     # mean |x|: fp32 tree on the GPU, fp64 on the host


def test_qsgd_same_random_stream():
    n, q = 128 * 512, 64
    dev, host = _pair({"compressor": "qsgd", "memory": "none", "communicator": "allgather", "quantum_num": q}, n,
                      steps=1)
    a, b = dev[0].view(-1, 128), host[0].view(-1, 128)
    diff = (a - b).abs()
    level = a.abs().max(dim=1).values.clamp_min(1e-12)[:, None]     # at least one level of the bucket
    assert float((diff > 1e-6 * level).float().mean()) < 0.01       # nearly all codes are the same
    g = torch.randn(n, generator=torch.Generator().manual_seed(0)) * 1e-3
    one_level = (g.view(-1, 128).norm(dim=1) / q)[:, None]
    assert bool((diff <= one_level * 1.01).all())                    # and no code is off by more than one level


def test_natural_compression_same_codes():
    for det in (True, False):
        dev, host = _pair({"compressor": "natural", "memory": "residual", "communicator": "allgather",
                           "deterministic": det}, 100_003, steps=3)
        for a, b in zip(dev, host):
            assert torch.equal(a, b)           # same Philox words, integer decisions: the same powers of two


def test_eight_bit_and_fp16_are_identical():
    dev, host = _pair({"compressor": "u8bit", "memory": "residual", "communicator": "allgather"}, 50_001, steps=2)
    assert all(torch.equal(a, b) for a, b in zip(dev, host))
    dev, host = _pair({"compressor": "fp16", "memory": "residual", "communicator": "allgather"}, 50_001, steps=2)
    assert all(torch.equal(a, b) for a, b in zip(dev, host))


def test_one_bit_and_terngrad_agree_to_rounding():
    dev, host = _pair({"compressor": "onebit", "memory": "none", "communicator": "allgather"}, 60_000, steps=1)
    torch.testing.assert_close(dev[0], host[0], rtol=1e-5, atol=1e-10)   # the two means: summed in another order
    dev, host = _pair({"compressor": "terngrad", "memory": "none", "communicator": "allgather"}, 60_000, steps=1)
    s = dev[0].abs().max()
    assert abs(float(s) - float(host[0].abs().max())) < 1e-6 * float(s)
    differ = ((dev[0] / s).round() != (host[0] / host[0].abs().max()).round()).float().mean()
    assert float(differ) < 0.005               # the scale differs in its last bits: a few keep decisions flip


def test_dgc_momentum_memory_small_and_large():
    for n in (5000, 150_000):                  # the single-CTA kernel and the large one
        dev, host = _pair({"compressor": "dgc", "memory": "dgc", "communicator": "allgather", "compress_ratio": 0.01,
                           "momentum": 0.9}, n, steps=3)
        for a, b in zip(dev, host):
            assert int((a != 0).sum()) == int((b != 0).sum()) == max(1, int(n * 0.01))
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-9)   # u = m u + g is one fused multiply-add on the GPU
